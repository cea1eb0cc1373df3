// Shared declarations of the CUDA backend: the device handle, error reporting, the launch
// counter and the small numeric helpers every kernel file uses.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/nuvec_cuda.h"

namespace nvc {

// ── errors ─────────────────────────────────────────────────────────────────────────────
int32_t set_error(int32_t status, const char *fmt, ...);
int32_t cuda_error(const char *call, cudaError_t err);

#define NVC_CUDA(call)                                                  \
    do {                                                                \
        cudaError_t err__ = (call);                                     \
        if (err__ != cudaSuccess) return nvc::cuda_error(#call, err__); \
    } while (0)

#define NVC_TRY(expr)                  \
    do {                               \
        int32_t rc__ = (expr);         \
        if (rc__ != NVC_OK) return rc__; \
    } while (0)

// ── caching device allocator (the reference's pool: crates/nuvec-gpu/src/cuda/memory.rs) ──
class Pool {
  public:
    int32_t alloc(size_t bytes, void **out);
    int32_t free(void *ptr);
    int32_t clear();
    void stats(nvc_mem_stats *out);
    void set_limit(uint64_t b) { std::lock_guard<std::mutex> g(mu_); limit_ = b; }
    void set_cache_limit(uint64_t b);
    void reset_peak() { std::lock_guard<std::mutex> g(mu_); peak_ = active_; }
    static size_t size_class(size_t bytes);

  private:
    void trim_locked(uint64_t target);
    std::mutex mu_;
    std::multimap<size_t, void *> free_;  // size class -> block
    std::map<void *, size_t> live_;       // block -> size class
    uint64_t active_ = 0, cached_ = 0, peak_ = 0, allocations_ = 0;
    uint64_t limit_ = ~0ull, cache_limit_ = ~0ull;
};

}  // namespace nvc

struct nvc_device {
    int ordinal = 0;
    cudaStream_t own_stream = nullptr;
    cudaStream_t stream = nullptr;
    cudaDeviceProp prop{};
    nvc::Pool pool;
    uint64_t launches = 0;
    bool capturing = false;   // between nvc_graph_begin and nvc_graph_end
    bool row_exact = false;   // nvc_set_row_exact: few-row products keep every row's one-row bits
    uint64_t captured = 0;    // kernels recorded by the open capture
    // Scratch owned by the handle and reused between calls (split-K partials and their
    // arrival counters); grown on demand from the pool.
    void *scratch = nullptr;
    size_t scratch_bytes = 0;
    uint32_t *counters = nullptr;  // zeroed; kernels leave them zeroed
    size_t counters_len = 0;
    // Pinned staging for the host-operand entry point.
    void *pinned = nullptr;
    size_t pinned_bytes = 0;
    void *staging = nullptr;
    size_t staging_bytes = 0;
    // Scratch of the tensor-core kernel's K-split tiles (partial tiles, arrival counters).
    void *qmm_partials = nullptr;
    size_t qmm_partials_bytes = 0;
    uint32_t *qmm_counters = nullptr;
    size_t qmm_counters_len = 0;
    // Host-mapped word a kernel sets when one of its bounded waits gives up; read at synchronisation.
    int32_t *error_word = nullptr, *error_word_dev = nullptr;
    // Asynchronous host-operand products: a pinned block (mapped into the device) and a device block
    // handed out front to back, and the results that wait in the pinned block for nvc_synchronize
    // to deliver them to the caller's memory.
    struct PendingResult { const void *pinned; void *host; size_t bytes; };
    std::mutex host_mu;
    std::vector<PendingResult> pending;
    char *ring_host = nullptr, *ring_host_dev = nullptr, *ring_dev = nullptr;  // (ring_host_dev: the pinned block as the device sees it)
    size_t ring_bytes = 0, ring_at = 0;
    // The last list given to nvc_quantized_matmul_host_batch: the second time the same list arrives
    // (same operands, sizes and host buffers, same place in the ring) its copy and kernels are
    // recorded, from the third on the recording is replayed.
    std::vector<unsigned char> batch_key;
    size_t batch_at = 0;
    cudaGraphExec_t batch_exec = nullptr;
    bool batch_norecord = false;  // this list failed to record once: it runs unrecorded
    uint64_t batch_kernels = 0;
    std::vector<PendingResult> batch_results;
};

struct nvc_graph {
    cudaGraphExec_t exec = nullptr;
    size_t nodes = 0;
    uint64_t kernels = 0;
};

struct nvc_event {
    cudaEvent_t ev = nullptr;
    int ordinal = 0;
};

namespace nvc {

int32_t make_current(nvc_device *dev);
int32_t ensure_scratch(nvc_device *dev, size_t bytes, void **out);
int32_t ensure_counters(nvc_device *dev, size_t count, uint32_t **out);
int32_t check_quant(const char *op, const nvc_quant *q);
int32_t check_launch(nvc_device *dev, const char *kernel);
// quantize.cu: bfloat16 x to nvfp4 / mxfp4 codes with the scales in the block-scaled MMA's layout (for qqmm.cu)
int32_t quantize_fp4_laid(nvc_device *dev, const nvc_quant *q, const void *x, int64_t rows, int64_t cols, uint32_t *codes, uint8_t *laid,
                          int64_t kblocks, int pieces);
int32_t deliver_pending(nvc_device *dev);    // copies finished host-operand results out (the stream must be idle)
int32_t ensure_error_word(nvc_device *dev);  // the host-mapped word kernels report a bounded wait's failure in

inline size_t dtype_size(int32_t dtype) { return dtype == NVC_F32 ? 4 : 2; }
inline bool is_float_dtype(int32_t d) { return d == NVC_F32 || d == NVC_F16 || d == NVC_BF16; }

// ── device-side numeric helpers ────────────────────────────────────────────────────────
template <typename T> struct DT;
template <> struct DT<float> {
    static __device__ __forceinline__ float load(const float *p, size_t i) { return p[i]; }
    static __device__ __forceinline__ float round(float x) { return x; }
    static __device__ __forceinline__ void store(float *p, size_t i, float x) { p[i] = x; }
};
template <> struct DT<__half> {
    static __device__ __forceinline__ float load(const __half *p, size_t i) { return __half2float(p[i]); }
    static __device__ __forceinline__ float round(float x) { return __half2float(__float2half_rn(x)); }
    static __device__ __forceinline__ void store(__half *p, size_t i, float x) { p[i] = __float2half_rn(x); }
};
template <> struct DT<__nv_bfloat16> {
    static __device__ __forceinline__ float load(const __nv_bfloat16 *p, size_t i) { return __bfloat162float(p[i]); }
    static __device__ __forceinline__ float round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
    static __device__ __forceinline__ void store(__nv_bfloat16 *p, size_t i, float x) { p[i] = __float2bfloat16_rn(x); }
};

// Code i of a little-endian stream of `bits`-bit values (the reference's packing,
// crates/nuvec-core/src/kernels.rs:749-756).
__device__ __forceinline__ uint32_t code_at(const uint8_t *bytes, size_t i, int bits) {
    size_t bit = i * (size_t)bits;
    size_t byte = bit >> 3;
    uint32_t shift = (uint32_t)(bit & 7);
    uint32_t v = (uint32_t)bytes[byte] >> shift;
    if (shift + bits > 8) v |= (uint32_t)bytes[byte + 1] << (8 - shift);
    return v & ((1u << bits) - 1u);
}

// float32 subnormals flushed to a signed zero (crates/nuvec-core/src/fp8.rs:107-113).
__device__ __forceinline__ float ftz(float x) {
    uint32_t u = __float_as_uint(x);
    return ((u & 0x7F800000u) == 0u) ? __uint_as_float(u & 0x80000000u) : x;
}
__device__ __forceinline__ float canonical(float x) { return x != x ? __uint_as_float(0x7FC00000u) : x; }

// E2M1 / E8M0 / E4M3 decoders (fp8.rs:39-44, 76-80, 96-102).
__device__ __forceinline__ float e2m1_to_f32(uint32_t code) {
    // magnitudes 0, .5, 1, 1.5, 2, 3, 4, 6
    uint32_t m = code & 7u;
    float v = m < 2u ? 0.5f * (float)m : (float)(2u + (m & 1u)) * __uint_as_float((125u + (m >> 1)) << 23);
    return (code & 8u) ? -v : v;
}
__device__ __forceinline__ float e8m0_to_f32(uint32_t code) {
    return code == 0u ? __uint_as_float(0x400000u) : __uint_as_float(code << 23);
}
__device__ __forceinline__ float e4m3_to_f32(uint32_t code) {
    uint32_t v = code & 127u;
    uint32_t e = v >> 3, m = v & 7u;
    float mag;
    if (v == 127u) mag = __uint_as_float(0x7FC00000u);
    else if (e == 0u) mag = (float)m * 0.001953125f;  // m * 2^-9
    else mag = __uint_as_float(((e + 120u) << 23) | (m << 20));
    return (code & 128u) ? -mag : mag;
}

}  // namespace nvc
