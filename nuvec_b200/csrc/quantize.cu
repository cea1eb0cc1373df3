// quantize / dequantize kernels: the parity gates of the path.
//
// Every rounding the reference's CPU kernels perform is performed here in the same order, so
// the outputs are equal bit for bit (crates/nuvec-core/src/kernels.rs:774-859 for affine,
// :914-1009 for mxfp4 / mxfp8 / nvfp4; codecs crates/nuvec-core/src/fp8.rs:18-129).
// Intrinsics with explicit rounding (__fmul_rn, __fadd_rn, __fdiv_rn) keep the compiler from
// contracting or approximating any step.
#include "common.cuh"

namespace nvc {

// ── dequantize ─────────────────────────────────────────────────────────────────────────

// Rows picked by index (an embedding look-up: QuantizedEmbedding::forward takes the ids' rows of
// the packed table, its scales and biases, then dequantizes them, crates/nuvec-nn/src/layers.rs:246-255):
// pack i of the output is pack `p` of source row ids[r]; an id past the end takes the last row, as
// `take` clamps (crates/nuvec-core/src/kernels.rs:120-133).  Without ids the source pack is i itself.
struct RowPick {
    const uint32_t *ids;   // nullptr: rows as they are
    size_t packs_per_row;  // cols / 8
    uint32_t rows;         // rows of the table
    __device__ __forceinline__ size_t source(size_t i) const {
        if (!ids) return i;
        const size_t r = i / packs_per_row, p = i - r * packs_per_row;
        return (size_t)min(ids[r], rows - 1u) * packs_per_row + p;
    }
};

// One thread decodes 8 consecutive values (8 * bits bits = `bits` whole bytes), which never
// straddle a group because every group size is a multiple of 8.
template <typename T, int BITS, bool FUSED>
__global__ void __launch_bounds__(256)
dequantize_affine_kernel(const uint8_t *__restrict__ codes, const T *__restrict__ scales,
                         const T *__restrict__ biases, T *__restrict__ out, size_t packs, int gs, RowPick pick) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= packs) return;
    const size_t si = pick.source(i);
    const uint8_t *src = codes + si * BITS;
    uint64_t stream = 0;
#pragma unroll
    for (int b = 0; b < BITS; b++) stream |= (uint64_t)src[b] << (8 * b);
    size_t first = i * 8;
    size_t g = si * 8 / (size_t)gs;
    float s = DT<T>::load(scales, g), bias = DT<T>::load(biases, g);
    float vals[8];
#pragma unroll
    for (int j = 0; j < 8; j++) {
        float c = (float)(uint32_t)((stream >> (j * BITS)) & ((1u << BITS) - 1u));
        if (FUSED) {
            vals[j] = __fmaf_rn(c, s, bias);  // rounded once on store
        } else {
            float p = DT<T>::round(__fmul_rn(c, s));  // product rounded to T
            vals[j] = __fadd_rn(p, bias);             // sum rounded to T on store
        }
    }
#pragma unroll
    for (int j = 0; j < 8; j++) DT<T>::store(out, first + j, vals[j]);
}

// Floating-point modes: BITS == 4 -> two E2M1 codes per byte, low nibble first; BITS == 8 ->
// one E4M3 code per byte.  One thread decodes 8 values.
template <typename T, int BITS>
__global__ void __launch_bounds__(256)
dequantize_fp_kernel(const uint8_t *__restrict__ codes, const uint8_t *__restrict__ scales,
                     const float *__restrict__ global, T *__restrict__ out, size_t packs, int gs, RowPick pick) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= packs) return;
    size_t first = i * 8;
    const size_t sfirst = pick.source(i) * 8;
    uint32_t sc = scales[sfirst / (size_t)gs];
    float scale = ftz(gs == 32 ? e8m0_to_f32(sc) : e4m3_to_f32(sc));
    if (global) {
        float inv = ftz(__fdiv_rn(*global, 448.0f * 6.0f));
        scale = ftz(__fmul_rn(scale, inv));
    }
#pragma unroll
    for (int j = 0; j < 8; j++) {
        float v;
        if (BITS == 8) v = e4m3_to_f32(codes[sfirst + j]);
        else v = e2m1_to_f32((codes[(sfirst + j) >> 1] >> (4 * (j & 1))) & 0xFu);
        DT<T>::store(out, first + j, canonical(ftz(__fmul_rn(scale, v))));
    }
}

template <typename T, bool FUSED>
static int32_t launch_dequantize_affine(nvc_device *dev, int bits, const uint8_t *codes, const void *scales,
                                        const void *biases, void *out, size_t packs, int gs, RowPick pick) {
    unsigned blocks = (unsigned)((packs + 255) / 256);
#define NVC_CASE(B)                                                                               \
    case B:                                                                                       \
        dequantize_affine_kernel<T, B, FUSED><<<blocks, 256, 0, dev->stream>>>(                   \
            codes, (const T *)scales, (const T *)biases, (T *)out, packs, gs, pick);              \
        break;
    switch (bits) {
        NVC_CASE(1) NVC_CASE(2) NVC_CASE(3) NVC_CASE(4) NVC_CASE(5) NVC_CASE(6) NVC_CASE(8)
    default: return set_error(NVC_ERR_INVALID_ARGUMENT, "dequantize: %d bits", bits);
    }
#undef NVC_CASE
    return check_launch(dev, "dequantize_affine_kernel");
}

// ── quantize ───────────────────────────────────────────────────────────────────────────

// One thread per group.  The arithmetic is float32 throughout, in the reference's order.
template <typename T>
__global__ void __launch_bounds__(128)
quantize_affine_kernel(const T *__restrict__ w, uint8_t *__restrict__ codes, T *__restrict__ scales,
                       T *__restrict__ biases, size_t groups, int gs, int bits) {
    size_t g = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (g >= groups) return;
    const size_t base = g * (size_t)gs;
    float lo = __int_as_float(0x7F800000), hi = __int_as_float(0xFF800000);
    for (int j = 0; j < gs; j++) {
        float v = DT<T>::load(w, base + j);
        lo = fminf(lo, v);
        hi = fmaxf(hi, v);
    }
    const float n_bins = (float)((1u << bits) - 1u), eps = 1e-7f;
    float scale, bias;
    if (bits == 1) {
        scale = fmaxf(__fsub_rn(hi, lo), eps);
        bias = lo;
    } else {
        bool wide = fabsf(lo) > fabsf(hi);
        scale = fmaxf(__fdiv_rn(__fsub_rn(hi, lo), n_bins), eps);
        scale = wide ? scale : -scale;
        float edge = wide ? lo : hi;
        float q0 = rintf(__fdiv_rn(edge, scale));
        if (q0 == 0.0f) {
            bias = 0.0f;
        } else {
            scale = __fdiv_rn(edge, q0);
            bias = edge;
        }
    }
    uint8_t *dst = codes + base * (size_t)bits / 8;
    uint64_t acc = 0;
    int have = 0;
    for (int j = 0; j < gs; j++) {
        float v = DT<T>::load(w, base + j);
        float r = rintf(__fdiv_rn(__fsub_rn(v, bias), scale));
        r = r < 0.0f ? 0.0f : (r > n_bins ? n_bins : r);
        uint32_t q = (r != r) ? 0u : (uint32_t)r;
        acc |= (uint64_t)q << have;
        have += bits;
        while (have >= 8) {
            *dst++ = (uint8_t)acc;
            acc >>= 8;
            have -= 8;
        }
    }
    DT<T>::store(scales, g, scale);
    DT<T>::store(biases, g, bias);
}

// fp8.rs:18-36
__device__ __forceinline__ uint32_t e4m3_from_f32(float x) {
    const uint32_t FP8_MAX = 543u << 21, DENORM_MASK = 141u << 23;
    uint32_t bits = __float_as_uint(x);
    uint32_t sign = bits & 0x80000000u;
    bits ^= sign;
    uint32_t code;
    if (bits >= FP8_MAX) {
        code = 0x7E;
    } else if (bits < (121u << 23)) {
        float sum = __fadd_rn(__uint_as_float(bits), __uint_as_float(DENORM_MASK));
        code = (__float_as_uint(sum) - DENORM_MASK) & 0xFFu;
    } else {
        uint32_t odd = (bits >> 20) & 1u;
        bits += ((uint32_t)(7 - 127) << 23) + 0x7FFFFu;
        bits += odd;
        code = (bits >> 20) & 0xFFu;
    }
    return code | (sign >> 24);
}

// fp8.rs:48-73
__device__ __forceinline__ uint32_t e2m1_from_f32(float x) {
    if (x != x) return 0x7u;
    uint32_t sign = (__float_as_uint(x) >> 31) ? 0x8u : 0x0u;
    float a = fabsf(x);
    uint32_t code = a > 5.0f ? 7u : a >= 3.5f ? 6u : a > 2.5f ? 5u : a >= 1.75f ? 4u
                  : a > 1.25f ? 3u : a >= 0.75f ? 2u : a > 0.25f ? 1u : 0u;
    return code | sign;
}

// Eight values to eight E2M1 codes in one word, value 0 in the low nibble, with the hardware's
// conversion: round to nearest even on the E2M1 grid, saturate at 6, NaN to +6 (code 7), the sign of
// a zero result kept: code for code the function above (fp8.rs:48-73; its thresholds 0.25, 0.75,
// 1.25, 1.75, 2.5, 3.5, 5 are the grid's ties, each going to the neighbour with an even mantissa).
__device__ __forceinline__ uint32_t e2m1x8_from_f32(const float *v) {
    uint32_t word;
    asm("{\n\t.reg .b8 c0, c1, c2, c3;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 c0, %2, %1;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 c1, %4, %3;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 c2, %6, %5;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 c3, %8, %7;\n\t"
        "mov.b32 %0, {c0, c1, c2, c3};\n\t}"
        : "=r"(word)
        : "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]));
    return word;
}

// The E8M0 code of mx_scale_round_up(x) for x >= 0 (fp8.rs:84-93, 124-130): the smallest
// power of two that is not below x, i.e. the exponent field, plus one when any mantissa bit
// is set, capped at 254; 0 for zero and 0xFF for Inf/NaN.
__device__ __forceinline__ uint32_t mx_scale_code(float x) {
    uint32_t u = __float_as_uint(x);
    uint32_t e = (u >> 23) & 0xFFu, m = u & 0x7FFFFFu;
    if (e == 0xFFu) return 0xFFu;
    if (e == 0u) return 0u;  // x was flushed: zero
    uint32_t code = e + (m != 0u ? 1u : 0u);
    return code > 254u ? 254u : code;
}

// LAID: the scales go straight into the block-scaled tensor-core layout of the qqmm kernel instead of the plain
// [rows, groups] array: 512-byte pieces of 128 rows x 4 scales, byte (r % 32) * 16 + (r % 128 / 32) * 4 + s,
// ordered [row tile][k-block of 256][piece]; the threads then cover the padded rows and groups too and write
// the padding's zero scales.
struct ScalePieces {
    uint8_t *out;
    int64_t rows, per_row, kblocks;
    int pieces;
};
template <typename T, int BITS, bool LAID = false>
__global__ void __launch_bounds__(128)
quantize_fp_kernel(const T *__restrict__ w, uint8_t *__restrict__ codes, uint8_t *__restrict__ scales,
                   const float *__restrict__ global, size_t groups, int gs, ScalePieces sp = ScalePieces{}) {
    size_t g = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t laid_at = 0;
    if (LAID) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the product kernel may set itself up meanwhile
    if (LAID) {
        const int64_t padded = sp.kblocks * sp.pieces * 4;  // groups per row, padding included
        const int64_t r = (int64_t)(g / (size_t)padded), gk = (int64_t)(g % (size_t)padded);
        if (r >= (sp.rows + 127) / 128 * 128) return;
        laid_at = (size_t)(((r / 128 * sp.kblocks + gk / (sp.pieces * 4)) * sp.pieces + (gk / 4) % sp.pieces) * 512 + (r % 32) * 16 +
                           (r % 128 / 32) * 4 + gk % 4);
        if (r >= sp.rows || gk >= sp.per_row) {
            sp.out[laid_at] = 0;
            return;
        }
        g = (size_t)(r * sp.per_row + gk);
    } else if (g >= groups) {
        return;
    }
    const size_t base = g * (size_t)gs;
    const bool mx = gs == 32;
    const float max_element = BITS == 4 ? 6.0f : 448.0f;
    const bool has = global != nullptr;
    const float scale_enc = has ? ftz(__fdiv_rn(448.0f * 6.0f, *global)) : 1.0f;
    // The group's values, once: 16-byte loads where the type and the alignment allow (the qqmm path
    // quantizes its activations with this kernel on every call), element by element otherwise.
    float vals[32];
    if (sizeof(T) == 2 && ((uintptr_t)(w + base) & 15) == 0) {
#pragma unroll
        for (int v4 = 0; v4 < 4; v4++) {
            if (8 * v4 >= gs) break;
            const uint4 raw = reinterpret_cast<const uint4 *>(w + base)[v4];
            const T *h = reinterpret_cast<const T *>(&raw);
#pragma unroll
            for (int e = 0; e < 8; e++) vals[8 * v4 + e] = ftz(DT<T>::load(h, e));
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; j++)
            if (j < gs) vals[j] = ftz(DT<T>::load(w, base + j));
    }
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < 32; j++)
        if (j < gs) amax = fmaxf(amax, fabsf(vals[j]));
    float scale = ftz(__fdiv_rn(amax, max_element));
    if (has) scale = ftz(__fmul_rn(scale, scale_enc));
    uint32_t code;
    float decoded;
    if (mx && !has) {
        code = mx_scale_code(scale);
        decoded = e8m0_to_f32(code);
    } else {
        code = e4m3_from_f32(scale);
        decoded = e4m3_to_f32(code);
    }
    if (LAID) sp.out[laid_at] = (uint8_t)code;
    else scales[g] = (uint8_t)code;
    decoded = ftz(decoded);
    float inverse = decoded == 0.0f ? 0.0f : ftz(__fdiv_rn(has ? scale_enc : 1.0f, decoded));
    if (BITS == 4) {
        // eight codes per 32-bit word, low nibble first; the group's words go out together
        uint32_t words[4] = {0u, 0u, 0u, 0u};
#pragma unroll
        for (int wd = 0; wd < 4; wd++) {
            if (8 * wd >= gs) break;
            float scaled[8];  // (a product below the normal range becomes a zero code either way)
#pragma unroll
            for (int e = 0; e < 8; e++) scaled[e] = __fmul_rn(vals[8 * wd + e], inverse);
            words[wd] = e2m1x8_from_f32(scaled);
        }
        uint32_t *dst = reinterpret_cast<uint32_t *>(codes + (base >> 1));  // (groups are multiples of 8 values: word-aligned)
        if (gs == 32 && ((uintptr_t)dst & 15) == 0) *reinterpret_cast<uint4 *>(dst) = make_uint4(words[0], words[1], words[2], words[3]);
        else if (gs == 16 && ((uintptr_t)dst & 7) == 0) *reinterpret_cast<uint2 *>(dst) = make_uint2(words[0], words[1]);
        else {
#pragma unroll
            for (int wd = 0; wd < 4; wd++)
                if (8 * wd < gs) dst[wd] = words[wd];
        }
    } else {
        // one byte per code: 16 of them to a store where the alignment allows
#pragma unroll
        for (int part = 0; part < 2; part++) {
            if (16 * part >= gs) break;
            uint32_t words[4];
#pragma unroll
            for (int wd = 0; wd < 4; wd++) {
                uint32_t word = 0;
#pragma unroll
                for (int e = 0; e < 4; e++)
                    word |= (uint32_t)e4m3_from_f32(canonical(ftz(__fmul_rn(vals[16 * part + 4 * wd + e], inverse)))) << (8 * e);
                words[wd] = word;
            }
            uint8_t *dst = codes + base + 16 * part;
            if (((uintptr_t)dst & 15) == 0) *reinterpret_cast<uint4 *>(dst) = make_uint4(words[0], words[1], words[2], words[3]);
            else {
#pragma unroll
                for (int j = 0; j < 16; j++) dst[j] = (uint8_t)(words[j >> 2] >> (8 * (j & 3)));
            }
        }
    }
}

template <typename T>
static int32_t quantize_typed(nvc_device *dev, const nvc_quant *q, const void *w, size_t count,
                              const float *global, uint32_t *codes, void *scales, void *biases) {
    size_t groups = count / (size_t)q->group_size;
    unsigned blocks = (unsigned)((groups + 127) / 128);
    if (q->mode == NVC_AFFINE) {
        quantize_affine_kernel<T><<<blocks, 128, 0, dev->stream>>>((const T *)w, (uint8_t *)codes, (T *)scales,
                                                                    (T *)biases, groups, q->group_size, q->bits);
        return check_launch(dev, "quantize_affine_kernel");
    }
    if (q->bits == 4)
        quantize_fp_kernel<T, 4><<<blocks, 128, 0, dev->stream>>>((const T *)w, (uint8_t *)codes, (uint8_t *)scales,
                                                                   global, groups, q->group_size);
    else
        quantize_fp_kernel<T, 8><<<blocks, 128, 0, dev->stream>>>((const T *)w, (uint8_t *)codes, (uint8_t *)scales,
                                                                   global, groups, q->group_size);
    return check_launch(dev, "quantize_fp_kernel");
}

template <typename T>
static int32_t dequantize_typed(nvc_device *dev, const nvc_quant *q, const uint32_t *codes, const void *scales,
                                const void *biases, const float *global, size_t count, void *out, int fused,
                                RowPick pick = RowPick{nullptr, 0, 0}) {
    size_t packs = count / 8;
    const uint8_t *bytes = (const uint8_t *)codes;
    if (q->mode == NVC_AFFINE) {
        return fused ? launch_dequantize_affine<T, true>(dev, q->bits, bytes, scales, biases, out, packs, q->group_size, pick)
                     : launch_dequantize_affine<T, false>(dev, q->bits, bytes, scales, biases, out, packs, q->group_size, pick);
    }
    unsigned blocks = (unsigned)((packs + 255) / 256);
    if (q->bits == 4)
        dequantize_fp_kernel<T, 4><<<blocks, 256, 0, dev->stream>>>(bytes, (const uint8_t *)scales, global, (T *)out, packs, q->group_size, pick);
    else
        dequantize_fp_kernel<T, 8><<<blocks, 256, 0, dev->stream>>>(bytes, (const uint8_t *)scales, global, (T *)out, packs, q->group_size, pick);
    return check_launch(dev, "dequantize_fp_kernel");
}

}  // namespace nvc

using namespace nvc;

extern "C" int32_t nvc_quantize(nvc_device *dev, const nvc_quant *q, int32_t dtype, const void *w, int64_t rows,
                                int64_t cols, const float *global_scale, uint32_t *out_codes, void *out_scales,
                                void *out_biases) {
    NVC_TRY(make_current(dev));
    NVC_TRY(check_quant("quantize", q));
    if (!is_float_dtype(dtype)) return set_error(NVC_ERR_UNSUPPORTED, "quantize: unsupported dtype %d", dtype);
    if (rows < 0 || cols < 0 || cols % q->group_size != 0)
        return set_error(NVC_ERR_INVALID_ARGUMENT,
                         "quantize: needs at least 2 dimensions with the last divisible by the group size %d, got [%lld, %lld]",
                         q->group_size, (long long)rows, (long long)cols);
    if (global_scale && q->mode != NVC_NVFP4)
        return set_error(NVC_ERR_INVALID_ARGUMENT, "quantize: a global scale is only supported for nvfp4");
    if (q->mode == NVC_AFFINE && !out_biases) return set_error(NVC_ERR_INVALID_ARGUMENT, "quantize: affine needs a biases output");
    size_t count = (size_t)rows * (size_t)cols;
    if (count == 0) return NVC_OK;
    if (!w || !out_codes || !out_scales) return set_error(NVC_ERR_INVALID_ARGUMENT, "quantize: null operand");
    switch (dtype) {
    case NVC_F32: return quantize_typed<float>(dev, q, w, count, global_scale, out_codes, out_scales, out_biases);
    case NVC_F16: return quantize_typed<__half>(dev, q, w, count, global_scale, out_codes, out_scales, out_biases);
    default: return quantize_typed<__nv_bfloat16>(dev, q, w, count, global_scale, out_codes, out_scales, out_biases);
    }
}

extern "C" int32_t nvc_dequantize(nvc_device *dev, const nvc_quant *q, int32_t dtype, const uint32_t *codes,
                                  const void *scales, const void *biases, const float *global_scale, int64_t rows,
                                  int64_t cols, void *out, int32_t fused) {
    NVC_TRY(make_current(dev));
    NVC_TRY(check_quant("dequantize", q));
    if (!is_float_dtype(dtype)) return set_error(NVC_ERR_UNSUPPORTED, "dequantize: unsupported dtype %d", dtype);
    if (q->mode == NVC_AFFINE && !biases)
        return set_error(NVC_ERR_INVALID_ARGUMENT, "dequantize: biases must be provided for affine quantization");
    if (q->mode != NVC_AFFINE && biases)
        return set_error(NVC_ERR_INVALID_ARGUMENT, "dequantize: biases must be null for this quantization mode");
    if (global_scale && q->mode != NVC_NVFP4)
        return set_error(NVC_ERR_INVALID_ARGUMENT, "dequantize: a global scale is only supported for nvfp4");
    if (rows < 0 || cols < 0 || cols % q->group_size != 0)
        return set_error(NVC_ERR_INVALID_ARGUMENT, "dequantize: %lld columns are not divisible by the group size %d",
                         (long long)cols, q->group_size);
    size_t count = (size_t)rows * (size_t)cols;
    if (count == 0) return NVC_OK;
    if (!codes || !scales || !out) return set_error(NVC_ERR_INVALID_ARGUMENT, "dequantize: null operand");
    switch (dtype) {
    case NVC_F32: return dequantize_typed<float>(dev, q, codes, scales, biases, global_scale, count, out, fused);
    case NVC_F16: return dequantize_typed<__half>(dev, q, codes, scales, biases, global_scale, count, out, fused);
    default: return dequantize_typed<__nv_bfloat16>(dev, q, codes, scales, biases, global_scale, count, out, fused);
    }
}

extern "C" int32_t nvc_quantized_embedding(nvc_device *dev, const nvc_quant *q, int32_t dtype, const uint32_t *codes, const void *scales,
                                           const void *biases, int64_t vocab, int64_t cols, const uint32_t *ids, int64_t count, void *out) {
    NVC_TRY(make_current(dev));
    NVC_TRY(check_quant("quantized_embedding", q));
    if (!is_float_dtype(dtype)) return set_error(NVC_ERR_UNSUPPORTED, "quantized_embedding: unsupported dtype %d", dtype);
    if (q->mode == NVC_AFFINE && !biases)
        return set_error(NVC_ERR_INVALID_ARGUMENT, "quantized_embedding: biases must be provided for affine quantization");
    if (q->mode != NVC_AFFINE && biases)
        return set_error(NVC_ERR_INVALID_ARGUMENT, "quantized_embedding: biases must be null for this quantization mode");
    if (vocab < 0 || count < 0 || cols < 0 || cols % q->group_size != 0 || vocab > 0xFFFFFFFFll)
        return set_error(NVC_ERR_INVALID_ARGUMENT, "quantized_embedding: invalid shape (%lld rows of %lld columns, group size %d)",
                         (long long)vocab, (long long)cols, q->group_size);
    const size_t total = (size_t)count * (size_t)cols;
    if (total == 0) return NVC_OK;
    if (vocab == 0) return set_error(NVC_ERR_INVALID_ARGUMENT, "quantized_embedding: rows taken from an empty table");
    if (!codes || !scales || !ids || !out) return set_error(NVC_ERR_INVALID_ARGUMENT, "quantized_embedding: null operand");
    const RowPick pick{ids, (size_t)cols / 8, (uint32_t)vocab};
    switch (dtype) {
    case NVC_F32: return dequantize_typed<float>(dev, q, codes, scales, biases, nullptr, total, out, 0, pick);
    case NVC_F16: return dequantize_typed<__half>(dev, q, codes, scales, biases, nullptr, total, out, 0, pick);
    default: return dequantize_typed<__nv_bfloat16>(dev, q, codes, scales, biases, nullptr, total, out, 0, pick);
    }
}

// The activation side of nvc_qqmm: bfloat16 x [rows, cols] to 4-bit codes (nvfp4 or mxfp4, no global scale) with the
// scales written straight into the tensor core's layout (laid: row_tiles x kblocks x pieces x 512 bytes).
int32_t nvc::quantize_fp4_laid(nvc_device *dev, const nvc_quant *q, const void *x, int64_t rows, int64_t cols, uint32_t *codes, uint8_t *laid,
                               int64_t kblocks, int pieces) {
    const int64_t padded_rows = (rows + 127) / 128 * 128, padded_groups = kblocks * pieces * 4;
    const size_t threads = (size_t)padded_rows * (size_t)padded_groups;
    ScalePieces sp{laid, rows, cols / q->group_size, kblocks, pieces};
    quantize_fp_kernel<__nv_bfloat16, 4, true><<<(unsigned)((threads + 127) / 128), 128, 0, dev->stream>>>(
        (const __nv_bfloat16 *)x, (uint8_t *)codes, nullptr, nullptr, 0, q->group_size, sp);
    return check_launch(dev, "quantize_fp_kernel");
}

// FastOp::QuantizeDequantize (crates/nuvec-core/src/products.rs:306-315, MLX's fp_quantize_dequantize): x through
// its quantization in a floating-point mode, the values the codes represent, in x's dtype -- the activation side of
// qqmm and gather_qqmm.  The reference's quantize followed by its dequantize; codes and scales pass through pool
// scratch (so not inside a recorded step).
extern "C" int32_t nvc_quantize_dequantize(nvc_device *dev, const nvc_quant *q, int32_t dtype, const void *x, int64_t rows, int64_t cols,
                                           const float *global_scale, void *out) {
    NVC_TRY(make_current(dev));
    NVC_TRY(check_quant("quantize_dequantize", q));
    if (q->mode == NVC_AFFINE) return set_error(NVC_ERR_INVALID_ARGUMENT, "quantize_dequantize: needs a floating-point mode (mxfp4, mxfp8 or nvfp4)");
    if (rows < 0 || cols < 0 || cols % q->group_size != 0) return set_error(NVC_ERR_INVALID_ARGUMENT, "quantize_dequantize: invalid shape");
    if (rows * cols == 0) return NVC_OK;
    if (dev->capturing) return set_error(NVC_ERR_UNSUPPORTED, "quantize_dequantize: not inside a recorded step (it takes scratch from the pool)");
    void *codes = nullptr, *scales = nullptr;
    NVC_TRY(dev->pool.alloc((size_t)rows * cols * q->bits / 8, &codes));
    int32_t rc = dev->pool.alloc((size_t)rows * (cols / q->group_size), &scales);
    if (rc == NVC_OK) rc = nvc_quantize(dev, q, dtype, x, rows, cols, global_scale, (uint32_t *)codes, scales, nullptr);
    if (rc == NVC_OK) rc = nvc_dequantize(dev, q, dtype, (const uint32_t *)codes, scales, nullptr, global_scale, rows, cols, out, 0);
    if (codes) dev->pool.free(codes);  // (the pool hands the blocks out again in stream order)
    if (scales) dev->pool.free(scales);
    return rc;
}
