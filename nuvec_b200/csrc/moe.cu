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
//               order, rounded once;
//   moe_sort    SwitchGlu::forward's bookkeeping for many rows (crates/nuvec-lm/src/model.rs:2199-2210): the
//               stable ascending argsort of the flattened expert indices (kernels.rs:231-266), its inverse
//               (the argsort of the argsort), each sorted pair's token (pair / k) and expert, and the
//               experts' first rows (sorted_offsets); integers throughout;
//   take_rows   `take(.., 0)` of whole rows (the activations by token, the results back into pair order),
//               indices past the end clamped (kernels.rs:120-133);
//   swiglu / swiglu_oai  the activation between the up/gate and the down products
//               (crates/nuvec-nn/src/lib.rs:513-579; SwitchGlu::through, model.rs:2160-2171): on the CPU the
//               compiled function is its operations one by one (crates/nuvec-core/src/fused.rs:214-217), each
//               rounded to the array's type, the sigmoid as MLX's (kernels.rs:1538-1543) in float32.  The
//               only step that is not an IEEE operation is the exponential: where the device's expf and the
//               host's differ in their last bit a result can differ by a unit or two in the last place;
//   rms_norm / add_rms_norm  fast::rms_norm and fast::add_rms_norm (fast/imp.rs:358-412), the normalisation in
//               front of a layer's projections, with the arithmetic of their CPU expansion
//               (fast/imp.rs:1367-1379): float32 squares, their sum in float64 over 8 lanes combined by a
//               fixed tree (kernels.rs:611-624) and rounded to float32, times float32(1 / d), plus eps,
//               1 / sqrt, x * that rounded to the array's type, times the weight rounded again; the sum
//               x + residual of add_rms_norm rounded to the type first.  Every step is an IEEE operation
//               performed in the reference's order: the results are its bits;
//   expert_bias_add  SwitchProjection::forward's `y.add(bias.take(indices, 0))`
//               (crates/nuvec-lm/src/model.rs:2139-2143): every gathered row plus its expert's bias,
//               float32 arithmetic for the halves, one rounding; an index past the end selects the
//               last expert (kernels.rs:120-133).
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

// Stable sort of `pairs` expert indices by one block.  A histogram and its exclusive scan give every
// expert its first place.  Then the pairs are taken 1024 at a time, one per thread: the lanes of a warp
// that hold the same expert rank themselves (__match_any_sync) and leave their number in a
// [warp][expert] table; a pair's place is its expert's next place, plus the table's entries of the
// warps before its own, plus its rank.  Warps and lanes follow the pairs' order, so an expert's pairs
// keep theirs: the reference's stable sort.  At most MOE_ROUTE_MAX experts.
__global__ void __launch_bounds__(1024) moe_sort_kernel(const uint32_t *__restrict__ indices, int64_t pairs, uint32_t k, uint32_t experts,
                                                        uint32_t *__restrict__ order, uint32_t *__restrict__ restore,
                                                        uint32_t *__restrict__ tokens, uint32_t *__restrict__ sorted,
                                                        int32_t *__restrict__ offsets) {
    __shared__ uint32_t next[MOE_ROUTE_MAX];          // expert -> its next place
    __shared__ uint8_t in_warp[32 * MOE_ROUTE_MAX];   // [warp][expert] (pitch `experts`): the expert's pairs among the warp's 32
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    for (uint32_t c = tid; c < experts; c += 1024u) next[c] = 0u;
    __syncthreads();
    for (int64_t i = tid; i < pairs; i += 1024) atomicAdd(&next[min(indices[i], experts - 1u)], 1u);
    __syncthreads();
    if (tid == 0) {
        uint32_t at = 0;
        for (uint32_t c = 0; c < experts; c++) {
            const uint32_t n = next[c];
            next[c] = at;
            if (offsets) offsets[c] = (int32_t)at;
            at += n;
        }
    }
    for (int64_t base = 0; base < pairs; base += 1024) {
        for (uint32_t c = tid; c < 32u * experts; c += 1024u) in_warp[c] = 0;
        __syncthreads();  // (also: the scan above, the previous round's update of `next`)
        const int64_t i = base + tid;
        const bool have = i < pairs;
        const uint32_t e = have ? min(indices[i], experts - 1u) : 0xFFFFFFFFu;
        const uint32_t peers = __match_any_sync(0xFFFFFFFFu, e);
        const uint32_t before = __popc(peers & ((1u << lane) - 1u));
        if (have && before == 0u) in_warp[warp * experts + e] = (uint8_t)__popc(peers);
        __syncthreads();
        if (have) {
            uint32_t pos = next[e] + before;
            for (uint32_t w = 0; w < warp; w++) pos += in_warp[w * experts + e];
            order[pos] = (uint32_t)i;
            restore[i] = pos;
            if (tokens) tokens[pos] = (uint32_t)(i / k);
            if (sorted) sorted[pos] = e;
        }
        __syncthreads();
        for (uint32_t c = tid; c < experts; c += 1024u) {
            uint32_t total = 0;
            for (uint32_t w = 0; w < 32u; w++) total += in_warp[w * experts + c];
            next[c] += total;
        }
        __syncthreads();
    }
}

// out[i, :] = src[min(idx[i], src_rows - 1), :], rows of row_bytes bytes; 16-byte pieces when everything is aligned.
__global__ void __launch_bounds__(256) take_rows_kernel(const uint8_t *__restrict__ src, int64_t src_rows, int64_t row_bytes,
                                                        const uint32_t *__restrict__ idx, uint8_t *__restrict__ out, int wide) {
    const int64_t i = blockIdx.x;
    const int64_t from = min((int64_t)idx[i], src_rows - 1);
    const uint8_t *a = src + from * row_bytes;
    uint8_t *b = out + i * row_bytes;
    if (wide) {
        for (int64_t c = threadIdx.x; c < row_bytes / 16; c += 256)
            reinterpret_cast<uint4 *>(b)[c] = reinterpret_cast<const uint4 *>(a)[c];
    } else {
        for (int64_t c = threadIdx.x; c < row_bytes; c += 256) b[c] = a[c];
    }
}

// MLX's Sigmoid in float32 (kernels.rs:1538-1543): y = 1 / (1 + exp(|x|)), then x < 0 ? y : 1 - y.
__device__ __forceinline__ float sigmoid_f32(float x) {
    const float a = x < 0.0f ? -x : x;
    const float y = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(a)));
    return x < 0.0f ? y : __fsub_rn(1.0f, y);
}
// minimum / maximum that propagate NaN (kernels.rs:1366-1367)
__device__ __forceinline__ float min_nan(float a, float b) { return (a != a || b != b) ? __int_as_float(0x7FC00000) : fminf(a, b); }
__device__ __forceinline__ float max_nan(float a, float b) { return (a != a || b != b) ? __int_as_float(0x7FC00000) : fmaxf(a, b); }

// out = silu(gate) * up, op by op: s = sigmoid(g), t = g * s, out = t * up, each rounded to T.
// OAI form (alpha, limit already rounded to T): g = min(gate, limit), x = min(max(up, -limit), limit),
// out = (x + 1) * (g * sigmoid(alpha * g)), each operation rounded to T.
template <typename T, bool OAI>
__global__ void __launch_bounds__(256) swiglu_kernel(const T *__restrict__ gate, const T *__restrict__ up, T *__restrict__ out, int64_t n,
                                                     float alpha, float limit) {
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= n) return;
    auto r = [](float v) { return Glue<T>::widen(Glue<T>::from_f32(v)); };  // one rounding to T
    float g = Glue<T>::load(gate, i), x = Glue<T>::load(up, i);
    if (OAI) {
        g = min_nan(g, limit);
        x = min_nan(max_nan(x, -limit), limit);
        const float s = r(sigmoid_f32(r(__fmul_rn(alpha, g))));
        const float gs = r(__fmul_rn(g, s));
        out[i] = Glue<T>::from_f32(__fmul_rn(r(__fadd_rn(x, 1.0f)), gs));
    } else {
        const float s = r(sigmoid_f32(g));
        const float t = r(__fmul_rn(g, s));
        out[i] = Glue<T>::from_f32(__fmul_rn(t, x));
    }
}

// One block per row.  The float64 lane sums must be taken in the reference's order (addition does
// not associate): threads 0-7 each add their lane's squares one after the other from shared memory.
template <typename T>
__global__ void __launch_bounds__(256) rms_norm_kernel(const T *__restrict__ x, const T *__restrict__ residual, const T *__restrict__ weight,
                                                       T *__restrict__ sum_out, T *__restrict__ y, int64_t d, float eps, float inv_count) {
    extern __shared__ float squares[];  // [d], then 8 lane sums (float64) and the scale
    double *lanes = reinterpret_cast<double *>(squares + ((d + 1) & ~(int64_t)1));
    float *scale = reinterpret_cast<float *>(lanes + 8);
    const int tid = threadIdx.x;
    const T *xr = x + (size_t)blockIdx.x * d;
    const T *rr = residual ? residual + (size_t)blockIdx.x * d : nullptr;
    T *hr = sum_out ? sum_out + (size_t)blockIdx.x * d : nullptr;
    T *yr = y + (size_t)blockIdx.x * d;
    for (int64_t j = tid; j < d; j += 256) {
        float v = Glue<T>::load(xr, j);
        if (rr) {
            const T h = Glue<T>::from_f32(__fadd_rn(v, Glue<T>::load(rr, j)));  // x + residual, rounded to T
            hr[j] = h;
            v = Glue<T>::widen(h);
        }
        squares[j] = __fmul_rn(v, v);
    }
    __syncthreads();
    if (tid < 8) {
        double acc = 0.0;
        const int64_t whole = d & ~(int64_t)7;
        for (int64_t j = tid; j < whole; j += 8) acc = __dadd_rn(acc, (double)squares[j]);
        if (tid < d - whole) acc = __dadd_rn(acc, (double)squares[whole + tid]);
        lanes[tid] = acc;
    }
    __syncthreads();
    if (tid == 0) {
        const double total = __dadd_rn(__dadd_rn(__dadd_rn(lanes[0], lanes[4]), __dadd_rn(lanes[1], lanes[5])),
                                       __dadd_rn(__dadd_rn(lanes[2], lanes[6]), __dadd_rn(lanes[3], lanes[7])));
        const float mean = __fmul_rn(__double2float_rn(total), inv_count);
        *scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
    }
    __syncthreads();
    const float n = *scale;
    for (int64_t j = tid; j < d; j += 256) {
        const float v = rr ? Glue<T>::widen(hr[j]) : Glue<T>::load(xr, j);
        T out = Glue<T>::from_f32(__fmul_rn(v, n));
        if (weight) out = Glue<T>::from_f32(__fmul_rn(Glue<T>::widen(out), Glue<T>::load(weight, j)));
        yr[j] = out;
    }
}

// y[r, c] += bias[indices[r], c]: one block per row; 16-byte pieces when the rows allow it.
template <typename T>
__global__ void __launch_bounds__(256) expert_bias_add_kernel(T *__restrict__ y, const T *__restrict__ bias,
                                                              const uint32_t *__restrict__ indices, int64_t n, uint32_t experts, int wide) {
    const int64_t r = blockIdx.x;
    const uint32_t e = min(indices[r], experts - 1u);
    T *row = y + r * n;
    const T *b = bias + (size_t)e * n;
    constexpr int PER = 16 / sizeof(T);
    if (wide) {
        for (int64_t c = threadIdx.x; c < n / PER; c += 256) {
            uint4 a = reinterpret_cast<uint4 *>(row)[c];
            const uint4 q = reinterpret_cast<const uint4 *>(b)[c];
            T *av = reinterpret_cast<T *>(&a);
            const T *qv = reinterpret_cast<const T *>(&q);
#pragma unroll
            for (int v = 0; v < PER; v++) av[v] = Glue<T>::from_f32(Glue<T>::widen(av[v]) + Glue<T>::widen(qv[v]));
            reinterpret_cast<uint4 *>(row)[c] = a;
        }
    } else {
        for (int64_t c = threadIdx.x; c < n; c += 256) row[c] = Glue<T>::from_f32(Glue<T>::widen(row[c]) + Glue<T>::load(b, c));
    }
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

extern "C" int32_t nvc_expert_bias_add(nvc_device *dev, int32_t dtype, void *y, const void *bias, const uint32_t *indices, int64_t rows,
                                       int64_t n, int64_t experts) {
    NVC_TRY(make_current(dev));
    if (!is_float_dtype(dtype)) return set_error(NVC_ERR_INVALID_ARGUMENT, "expert_bias_add: y must be floating point (dtype %d)", dtype);
    if (rows < 0 || n < 0 || experts < 0 || experts > 0xFFFFFFFFll) return set_error(NVC_ERR_INVALID_ARGUMENT, "expert_bias_add: invalid shape");
    if (rows * n == 0) return NVC_OK;
    if (experts == 0) return set_error(NVC_ERR_INVALID_ARGUMENT, "expert_bias_add: no experts to take a bias from");
    if (!y || !bias || !indices) return set_error(NVC_ERR_INVALID_ARGUMENT, "expert_bias_add: null operand");
    if (rows > 0x7FFFFFFFll) return set_error(NVC_ERR_UNSUPPORTED, "expert_bias_add: %lld rows exceed the grid limit", (long long)rows);
    const size_t item = dtype == NVC_F32 ? 4 : 2;
    const int wide = (n * item) % 16 == 0 && (uintptr_t)y % 16 == 0 && (uintptr_t)bias % 16 == 0;
    switch (dtype) {
    case NVC_F32:
        expert_bias_add_kernel<float><<<(unsigned)rows, 256, 0, dev->stream>>>((float *)y, (const float *)bias, indices, n, (uint32_t)experts, wide);
        break;
    case NVC_F16:
        expert_bias_add_kernel<__half><<<(unsigned)rows, 256, 0, dev->stream>>>((__half *)y, (const __half *)bias, indices, n, (uint32_t)experts, wide);
        break;
    default:
        expert_bias_add_kernel<__nv_bfloat16><<<(unsigned)rows, 256, 0, dev->stream>>>((__nv_bfloat16 *)y, (const __nv_bfloat16 *)bias, indices, n,
                                                                                     (uint32_t)experts, wide);
    }
    return check_launch(dev, "expert_bias_add_kernel");
}

extern "C" int32_t nvc_moe_sort(nvc_device *dev, const uint32_t *indices, int64_t pairs, int64_t k, int64_t experts, uint32_t *out_order,
                                uint32_t *out_restore, uint32_t *out_tokens, uint32_t *out_sorted, int32_t *out_offsets) {
    NVC_TRY(make_current(dev));
    if (pairs < 0 || k < 1 || experts < 0 || pairs > 0x7FFFFFFFll) return set_error(NVC_ERR_INVALID_ARGUMENT, "moe_sort: invalid shape");
    if (experts > MOE_ROUTE_MAX) return set_error(NVC_ERR_UNSUPPORTED, "moe_sort: %lld experts (at most %d)", (long long)experts, MOE_ROUTE_MAX);
    if (pairs > 0 && experts == 0) return set_error(NVC_ERR_INVALID_ARGUMENT, "moe_sort: pairs without experts");
    if (pairs == 0 && experts == 0) return NVC_OK;
    if ((pairs > 0 && (!indices || !out_order || !out_restore))) return set_error(NVC_ERR_INVALID_ARGUMENT, "moe_sort: null operand");
    moe_sort_kernel<<<1, 1024, 0, dev->stream>>>(indices, pairs, (uint32_t)k, (uint32_t)experts, out_order, out_restore, out_tokens, out_sorted,
                                                 out_offsets);
    return check_launch(dev, "moe_sort_kernel");
}

extern "C" int32_t nvc_take_rows(nvc_device *dev, const void *src, int64_t src_rows, int64_t row_bytes, const uint32_t *indices, int64_t n,
                                 void *out) {
    NVC_TRY(make_current(dev));
    if (src_rows < 0 || row_bytes < 0 || n < 0 || n > 0x7FFFFFFFll) return set_error(NVC_ERR_INVALID_ARGUMENT, "take_rows: invalid shape");
    if (n * row_bytes == 0) return NVC_OK;
    if (src_rows == 0) return set_error(NVC_ERR_INVALID_ARGUMENT, "take_rows: rows taken from an empty array");
    if (!src || !indices || !out) return set_error(NVC_ERR_INVALID_ARGUMENT, "take_rows: null operand");
    const int wide = row_bytes % 16 == 0 && (uintptr_t)src % 16 == 0 && (uintptr_t)out % 16 == 0;
    take_rows_kernel<<<(unsigned)n, 256, 0, dev->stream>>>((const uint8_t *)src, src_rows, row_bytes, indices, (uint8_t *)out, wide);
    return check_launch(dev, "take_rows_kernel");
}

template <bool OAI>
static int32_t launch_swiglu(nvc_device *dev, const char *op, int32_t dtype, const void *gate, const void *up, int64_t n, float alpha,
                             float limit, void *out) {
    NVC_TRY(make_current(dev));
    if (!is_float_dtype(dtype)) return set_error(NVC_ERR_INVALID_ARGUMENT, "%s: operands must be floating point (dtype %d)", op, dtype);
    if (n < 0) return set_error(NVC_ERR_INVALID_ARGUMENT, "%s: invalid size", op);
    if (n == 0) return NVC_OK;
    if (!gate || !up || !out) return set_error(NVC_ERR_INVALID_ARGUMENT, "%s: null operand", op);
    const int64_t blocks = (n + 255) / 256;
    if (blocks > 0x7FFFFFFFll) return set_error(NVC_ERR_UNSUPPORTED, "%s: %lld elements exceed the grid limit", op, (long long)n);
    switch (dtype) {
    case NVC_F32:
        swiglu_kernel<float, OAI><<<(unsigned)blocks, 256, 0, dev->stream>>>((const float *)gate, (const float *)up, (float *)out, n, alpha, limit);
        break;
    case NVC_F16:
        // (the scalars are weak: rounded to the arrays' type, crates/nuvec-nn/src/lib.rs:504-507)
        swiglu_kernel<__half, OAI><<<(unsigned)blocks, 256, 0, dev->stream>>>((const __half *)gate, (const __half *)up, (__half *)out, n,
                                                                             __half2float(__float2half_rn(alpha)), __half2float(__float2half_rn(limit)));
        break;
    default:
        swiglu_kernel<__nv_bfloat16, OAI><<<(unsigned)blocks, 256, 0, dev->stream>>>(
            (const __nv_bfloat16 *)gate, (const __nv_bfloat16 *)up, (__nv_bfloat16 *)out, n, __bfloat162float(__float2bfloat16_rn(alpha)),
            __bfloat162float(__float2bfloat16_rn(limit)));
    }
    return check_launch(dev, "swiglu_kernel");
}

extern "C" int32_t nvc_swiglu(nvc_device *dev, int32_t dtype, const void *gate, const void *up, int64_t n, void *out) {
    return launch_swiglu<false>(dev, "swiglu", dtype, gate, up, n, 0.0f, 0.0f, out);
}

extern "C" int32_t nvc_swiglu_oai(nvc_device *dev, int32_t dtype, const void *gate, const void *up, float alpha, float limit, int64_t n,
                                  void *out) {
    return launch_swiglu<true>(dev, "swiglu_oai", dtype, gate, up, n, alpha, limit, out);
}

static int32_t launch_rms_norm(nvc_device *dev, const char *op, int32_t dtype, const void *x, const void *residual, const void *weight, float eps,
                               int64_t rows, int64_t d, void *sum_out, void *y) {
    NVC_TRY(make_current(dev));
    if (!is_float_dtype(dtype)) return set_error(NVC_ERR_INVALID_ARGUMENT, "%s: the input must be floating point (dtype %d)", op, dtype);
    if (rows < 0 || d < 0 || rows > 0x7FFFFFFFll) return set_error(NVC_ERR_INVALID_ARGUMENT, "%s: invalid shape", op);
    if (rows * d == 0) return NVC_OK;
    if (!x || !y || (residual && !sum_out)) return set_error(NVC_ERR_INVALID_ARGUMENT, "%s: null operand", op);
    const size_t smem = (size_t)((d + 1) & ~(int64_t)1) * sizeof(float) + 8 * sizeof(double) + 16;
    if (smem > 200 * 1024) return set_error(NVC_ERR_UNSUPPORTED, "%s: rows of %lld elements do not fit shared memory", op, (long long)d);
    const float inv_count = (float)(1.0 / (double)d);
#define NVC_RMS(T)                                                                                                              \
    {                                                                                                                           \
        auto kernel = rms_norm_kernel<T>;                                                                                       \
        static bool configured[64] = {};                                                                                        \
        if (smem > 48 * 1024 && dev->ordinal >= 0 && dev->ordinal < 64 && !configured[dev->ordinal]) {                          \
            NVC_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));                    \
            configured[dev->ordinal] = true;                                                                                    \
        }                                                                                                                       \
        kernel<<<(unsigned)rows, 256, smem, dev->stream>>>((const T *)x, (const T *)residual, (const T *)weight, (T *)sum_out, (T *)y, d, eps, \
                                                           inv_count);                                                          \
    }
    switch (dtype) {
    case NVC_F32: NVC_RMS(float) break;
    case NVC_F16: NVC_RMS(__half) break;
    default: NVC_RMS(__nv_bfloat16)
    }
#undef NVC_RMS
    return check_launch(dev, "rms_norm_kernel");
}

extern "C" int32_t nvc_rms_norm(nvc_device *dev, int32_t dtype, const void *x, const void *weight, float eps, int64_t rows, int64_t d, void *y) {
    return launch_rms_norm(dev, "rms_norm", dtype, x, nullptr, weight, eps, rows, d, nullptr, y);
}

extern "C" int32_t nvc_add_rms_norm(nvc_device *dev, int32_t dtype, const void *x, const void *residual, const void *weight, float eps,
                                    int64_t rows, int64_t d, void *out_sum, void *y) {
    if (!residual) return set_error(NVC_ERR_INVALID_ARGUMENT, "add_rms_norm: null residual");
    return launch_rms_norm(dev, "add_rms_norm", dtype, x, residual, weight, eps, rows, d, out_sum, y);
}
