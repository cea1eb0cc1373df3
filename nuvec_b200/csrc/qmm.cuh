// Many-row quantized products (prefill, grouped mixture-of-experts) on tcgen05 (qmm.cu).
#pragma once
#include "common.cuh"

namespace nvc {

struct QmmParams {
    int32_t mode, gs, bits;
    const void *x;          // bf16 [rows, K] (row stride ldx)
    const uint32_t *w;      // [experts or 1][N, K*bits/32]
    const void *scales, *biases;
    const float *global;    // nullptr, one value, or one per expert
    int32_t expert_global;
    const int32_t *offsets; // grouped: first row of every expert (int32 [experts]); nullptr = one matrix
    int64_t experts;
    int64_t rows, N, K, ldx;
    void *y;                // bf16 [rows, N]
};
bool qmm_eligible(int32_t mode, int32_t gs, int32_t bits, int32_t dtype, int32_t transpose, int64_t M, int64_t N,
                  int64_t K, const void *x, int64_t ldx, const uint32_t *w);
int32_t launch_qmm(nvc_device *dev, const QmmParams &p);

}  // namespace nvc
