// The glue around a mixture of experts' products: the router's top-k selection with
// renormalisation and the weighted sum of the experts' outputs
// (fast::moe_route, fast::weighted_sum: crates/nuvec-core/src/fast/imp.rs:2652-2672, 2731-2747;
// their Metal kernels: crates/nuvec-kernels/src/metal/moe.metal).  Each kernel performs the
// arithmetic of the composition it stands for, in the order the reference's CPU path performs it
// (fast/imp.rs:1586-1600 over kernels.rs:231-273, 609-645, 1191-1195, 1581), so the results are
// the reference's bits:
//   moe_route   stable ascending order of a row's probabilities (NaN last), the last k indices,
//               their values, and with `normalize` those divided by their sum -- the sum taken in
//               float64 over 8 lanes combined by a fixed tree, rounded to the array's type, the
//               divide element-wise in that type (float32 arithmetic for the halves);
//   weighted_sum  the products x * w rounded to the array's type, summed over k in float64 in
//               order, rounded once.
#include "common.cuh"

namespace nvc {

template <typename T> struct Glue;
template <> struct Glue<float> {
    static __device__ __forceinline__ float load(const float *p, size_t i) { return p[i]; }
    static __device__ __forceinline__ float from_f32(float x) { return x; }
    static __device__ __forceinline__ float from_f64(double x) { return (float)x; }
    static __device__ __forceinline__ float widen(float x) { return x; }
};
template <> struct Glue<__half> {
    static __device__ __forceinline__ float load(const __half *p, size_t i) { return __half2float(p[i]); }
    static __device__ __forceinline__ __half from_f32(float x) { return __float2half_rn(x); }
    static __device__ __forceinline__ __half from_f64(double x) { return __double2half(x); }  // one rounding from float64
    static __device__ __forceinline__ float widen(__half x) { return __half2float(x); }
};
template <> struct Glue<__nv_bfloat16> {
    static __device__ __forceinline__ float load(const __nv_bfloat16 *p, size_t i) { return __bfloat162float(p[i]); }
    static __device__ __forceinline__ __nv_bfloat16 from_f32(float x) { return __float2bfloat16_rn(x); }
    // bfloat16 from float64 goes through float32 (crates/nuvec-core/src/cast.rs:84-96)
    static __device__ __forceinline__ __nv_bfloat16 from_f64(double x) { return __float2bfloat16_rn((float)x); }
    static __device__ __forceinline__ float widen(__nv_bfloat16 x) { return __bfloat162float(x); }
};

constexpr int MOE_ROUTE_MAX = 1024;  // one thread per expert

__device__ __forceinline__ bool route_less(float x, float y) {
    const bool xn = x != x, yn = y != y;
    if (!xn && !yn) return x < y;
    return !xn && yn;
}

// One block per row, one thread per expert: an expert's position in the sorted row is the number
// of experts that sort before it.
template <typename T>
__global__ void __launch_bounds__(MOE_ROUTE_MAX) moe_route_kernel(const T *__restrict__ probs, uint32_t *__restrict__ indices,
                                                                  T *__restrict__ scores, int experts, int k, int normalize) {
    __shared__ float p[MOE_ROUTE_MAX];
    __shared__ float top[MOE_ROUTE_MAX];
    __shared__ float total;
    const int e = threadIdx.x;
    const size_t row = blockIdx.x;
    if (e < experts) p[e] = Glue<T>::load(probs, row * experts + e);
    __syncthreads();
    if (e < experts) {
        const float v = p[e];
        int rank = 0;
        for (int j = 0; j < experts; j++) {
            const float u = p[j];
            rank += (route_less(u, v) || (!route_less(v, u) && j < e)) ? 1 : 0;
        }
        const int slot = rank - (experts - k);
        if (slot >= 0) {
            indices[row * k + slot] = (uint32_t)e;
            top[slot] = v;
        }
    }
    __syncthreads();
    if (normalize) {
        if (e == 0) {
            double acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            for (int j = 0; j < k; j++) acc[j & 7] += (double)top[j];
            const double sum = 0.0 + (((acc[0] + acc[4]) + (acc[1] + acc[5])) + ((acc[2] + acc[6]) + (acc[3] + acc[7])));
            total = Glue<T>::widen(Glue<T>::from_f64(sum));
        }
        __syncthreads();
        if (e < k) scores[row * k + e] = Glue<T>::from_f32(__fdiv_rn(top[e], total));
    } else if (e < k) {
        scores[row * k + e] = Glue<T>::from_f32(top[e]);
    }
}

// One thread per output element (row r, column c).
template <typename T>
__global__ void __launch_bounds__(256) weighted_sum_kernel(const T *__restrict__ x, const T *__restrict__ w, T *__restrict__ out,
                                                           int64_t rows, int k, int64_t d) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * d) return;
    const int64_t r = i / d, c = i - r * d;
    double s = 0.0;
    for (int j = 0; j < k; j++) {
        const float prod = __fmul_rn(Glue<T>::load(x, (size_t)((r * k + j) * d + c)), Glue<T>::load(w, (size_t)(r * k + j)));
        s += (double)Glue<T>::widen(Glue<T>::from_f32(prod));
    }
    out[i] = Glue<T>::from_f64(s);
}

}  // namespace nvc

using namespace nvc;

extern "C" int32_t nvc_moe_route(nvc_device *dev, int32_t dtype, const void *probs, int64_t rows, int64_t experts, int64_t k,
                                 int32_t normalize, uint32_t *out_indices, void *out_scores) {
    NVC_TRY(make_current(dev));
    if (!is_float_dtype(dtype)) return set_error(NVC_ERR_INVALID_ARGUMENT, "moe_route: probabilities must be floating point (dtype %d)", dtype);
    if (rows < 0 || experts < 0) return set_error(NVC_ERR_INVALID_ARGUMENT, "moe_route: negative size");
    if (k < 1 || k > experts)
        return set_error(NVC_ERR_INVALID_ARGUMENT, "moe_route: k must be in 1..=%lld for probabilities of %lld experts", (long long)experts,
                         (long long)experts);
    if (experts > MOE_ROUTE_MAX)
        return set_error(NVC_ERR_UNSUPPORTED, "moe_route: %lld experts (at most %d)", (long long)experts, MOE_ROUTE_MAX);
    if (rows == 0) return NVC_OK;
    if (!probs || !out_indices || !out_scores) return set_error(NVC_ERR_INVALID_ARGUMENT, "moe_route: null operand");
    if (rows > 0x7FFFFFFFll) return set_error(NVC_ERR_UNSUPPORTED, "moe_route: %lld rows exceed the grid limit", (long long)rows);
    const unsigned threads = (unsigned)((experts + 31) / 32 * 32);
    switch (dtype) {
    case NVC_F32:
        moe_route_kernel<float><<<(unsigned)rows, threads, 0, dev->stream>>>((const float *)probs, out_indices, (float *)out_scores,
                                                                            (int)experts, (int)k, normalize);
        break;
    case NVC_F16:
        moe_route_kernel<__half><<<(unsigned)rows, threads, 0, dev->stream>>>((const __half *)probs, out_indices, (__half *)out_scores,
                                                                             (int)experts, (int)k, normalize);
        break;
    default:
        moe_route_kernel<__nv_bfloat16><<<(unsigned)rows, threads, 0, dev->stream>>>((const __nv_bfloat16 *)probs, out_indices,
                                                                                    (__nv_bfloat16 *)out_scores, (int)experts, (int)k, normalize);
    }
    return check_launch(dev, "moe_route_kernel");
}

extern "C" int32_t nvc_weighted_sum(nvc_device *dev, int32_t dtype, const void *x, const void *w, int64_t rows, int64_t k, int64_t d,
                                    void *out) {
    NVC_TRY(make_current(dev));
    if (!is_float_dtype(dtype)) return set_error(NVC_ERR_INVALID_ARGUMENT, "weighted_sum: x must be floating point (dtype %d)", dtype);
    if (rows < 0 || k < 0 || d < 0 || k > 0x7FFFFFFFll) return set_error(NVC_ERR_INVALID_ARGUMENT, "weighted_sum: invalid shape");
    if (rows * d == 0) return NVC_OK;
    if (!out || (k > 0 && (!x || !w))) return set_error(NVC_ERR_INVALID_ARGUMENT, "weighted_sum: null operand");
    const int64_t blocks = (rows * d + 255) / 256;
    if (blocks > 0x7FFFFFFFll) return set_error(NVC_ERR_UNSUPPORTED, "weighted_sum: %lld outputs exceed the grid limit", (long long)(rows * d));
    switch (dtype) {
    case NVC_F32:
        weighted_sum_kernel<float><<<(unsigned)blocks, 256, 0, dev->stream>>>((const float *)x, (const float *)w, (float *)out, rows, (int)k, d);
        break;
    case NVC_F16:
        weighted_sum_kernel<__half><<<(unsigned)blocks, 256, 0, dev->stream>>>((const __half *)x, (const __half *)w, (__half *)out, rows, (int)k, d);
        break;
    default:
        weighted_sum_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, dev->stream>>>((const __nv_bfloat16 *)x, (const __nv_bfloat16 *)w,
                                                                                     (__nv_bfloat16 *)out, rows, (int)k, d);
    }
    return check_launch(dev, "weighted_sum_kernel");
}
