/*
 * CPU oracle for nuvec's quantized-matmul path.  TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of the reference's CPU implementation of quantize, dequantize,
 * quantized_matmul, gather_qmm and sorted_offsets.  It exists so the CUDA kernels can be
 * checked against the reference's arithmetic where the reference itself (Rust) cannot be
 * built.  Only the tests, the smoke check and the CPU-baseline leg of the benchmark may
 * call it; the CUDA library never links or loads it.
 *
 * Parity status: PINNED for quantize/dequantize (bit for bit against the reference's recorded
 * MLX vectors) and for products of up to 16 rows (summation order specified in the reference
 * tree).  Products of more than 16 rows go through the third-party `gemm` crate 0.19.0 in
 * the reference, whose summation order is not part of the reference tree: there the oracle
 * uses its own blocked f32 GEMM and parity is by tolerance only.
 *
 * Every function cites the reference lines it restates (paths inside hupe1980/nuvec).
 */
#ifndef NUVEC_ORACLE_H
#define NUVEC_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* dtype codes follow nuvec's DType order (crates/nuvec-core/tests/common/fixture.rs:14-29). */
enum { ORC_U8 = 1, ORC_U32 = 3, ORC_F16 = 9, ORC_BF16 = 10, ORC_F32 = 11 };
/* Quantization modes (crates/nuvec-core/src/quantized.rs:24-35). */
enum { ORC_AFFINE = 0, ORC_MXFP4 = 1, ORC_MXFP8 = 2, ORC_NVFP4 = 3 };

/* Codecs, crates/nuvec-core/src/fp8.rs:18-129. */
uint8_t orc_e4m3_from_f32(float x);
float orc_e4m3_to_f32(uint8_t code);
uint8_t orc_e2m1_from_f32(float x);
float orc_e2m1_to_f32(uint8_t code);
uint8_t orc_e8m0_from_f32(float x);
float orc_e8m0_to_f32(uint8_t code);
float orc_mx_scale_round_up(float x);

/* Scalar conversions used by every function here (crates/nuvec-core/src/cast.rs:70-98). */
uint16_t orc_f32_to_bf16(float x);
float orc_bf16_to_f32(uint16_t h);
uint16_t orc_f64_to_f16(double x);
float orc_f16_to_f32(uint16_t h);

/* Returns 0 on success, a negative value for an invalid combination (message via
 * orc_last_error). */
const char *orc_last_error(void);

/* Validates (mode, group_size, bits): crates/nuvec-core/src/quantized.rs:137-167. */
int orc_check_quant(int mode, int group_size, int bits);

/* kernels.rs:774-831 (affine) and :914-971 (mxfp4/mxfp8/nvfp4).  `w` is [rows, cols] of
 * `dtype`; scales/biases come back in `dtype` (affine) or as uint8 codes (fp modes, no
 * biases).  `global_scale` may be NULL (nvfp4 only otherwise). */
int orc_quantize(int mode, int group_size, int bits, int dtype, const void *w, size_t rows,
                 size_t cols, const float *global_scale, uint32_t *codes, void *scales,
                 void *biases);

/* kernels.rs:835-859 (affine: two roundings to the scales' dtype; `fused` != 0 gives the
 * Metal kernel's single rounding of fma(code, scale, bias), quantized.h:2701-2705) and
 * kernels.rs:976-1009 (fp modes, out_dtype in {f16,bf16,f32}). */
int orc_dequantize(int mode, int group_size, int bits, int dtype, const uint32_t *codes,
                   const void *scales, const void *biases, const float *global_scale,
                   size_t rows, size_t cols, void *out, int fused);

/* kernels.rs:875-892. */
int orc_sorted_offsets(const uint32_t *indices, size_t rows, size_t groups, int32_t *out);

/* kernels.rs:1091-1142 with the f32 product of nuvec-cpu (few_rows.rs:65-224 for M <= 16).
 * x is [M, K] of `dtype`; transposed weights are [N, K*bits/32], untransposed [K, N*bits/32].
 * flags bit 0: dequantize with all threads (the reference's loop is serial). */
int orc_quantized_matmul(int mode, int group_size, int bits, int dtype, int transpose,
                         const void *x, const uint32_t *w, const void *scales,
                         const void *biases, const float *global_scale, size_t M, size_t N,
                         size_t K, void *y, int flags);

/* quantized.rs:679-719: batch i is x[lhs[i]] (an [M, K] block) times expert rhs[i].
 * `global_scale` is [experts] or NULL. */
int orc_gather_qmm(int mode, int group_size, int bits, int dtype, int transpose, const void *x,
                   const uint32_t *w, const void *scales, const void *biases,
                   const float *global_scale, const uint32_t *lhs, const uint32_t *rhs,
                   size_t batches, size_t M, size_t N, size_t K, size_t experts, void *y,
                   int flags);

/* The f32 product alone (x [M,K] row-major, w [N,K] row-major): few_rows order for M <= 16. */
void orc_matmul_nt_f32(const float *x, const float *w, size_t M, size_t N, size_t K, float *y);

/* fast::moe_route / fast::weighted_sum (crates/nuvec-core/src/fast/imp.rs:2652-2672, 2731-2747) as their
 * CPU compositions compute them.  probs [rows, experts] -> indices u32 [rows, k] (ascending by
 * probability, stable), scores [rows, k];  x [rows, k, d], w [rows, k] -> out [rows, d]. */
int orc_moe_route(int dtype, const void *probs, size_t rows, size_t experts, size_t k, int normalize,
                  uint32_t *out_indices, void *out_scores);
int orc_weighted_sum(int dtype, const void *x, const void *w, size_t rows, size_t k, size_t d, void *out);
int orc_expert_bias_add(int dtype, void *y, const void *bias, const uint32_t *indices, size_t rows, size_t n, size_t experts);
int orc_moe_sort(const uint32_t *indices, size_t pairs, size_t k, size_t experts, uint32_t *order, uint32_t *restore,
                 uint32_t *tokens, uint32_t *sorted, int32_t *offsets);
int orc_swiglu(int dtype, int oai, const void *gate, const void *up, float alpha, float limit, size_t n, void *out);
int orc_rms_norm(int dtype, const void *x, const void *residual, const void *weight, float eps, size_t rows, size_t d, void *sum_out,
                 void *y);
int orc_threads(void);
void orc_set_threads(int n);

#ifdef __cplusplus
}
#endif
#endif
