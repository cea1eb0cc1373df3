/*
 * CPU oracle for nuvec's quantized-matmul path.  TEST INFRASTRUCTURE ONLY -- see
 * nuvec_oracle.h for what may call it and for the parity status.
 *
 * Build: gcc -O3 -march=native -ffp-contract=off -fopenmp -fPIC -shared (see Makefile).
 * Floating-point contraction is off so that every rounding written here happens; fused
 * multiply-adds are spelled fmaf() where the reference uses mul_add.
 */
#include "nuvec_oracle.h"

#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static _Thread_local char g_error[256];

const char *orc_last_error(void) { return g_error; }

static int fail(const char *fmt, long a, long b) {
    snprintf(g_error, sizeof g_error, fmt, a, b);
    return -1;
}

int orc_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Threads the parallel parts use from now on (launchers such as torchrun export OMP_NUM_THREADS=1;
 * the timed CPU arm asks for the host's cores explicitly, as the reference's rayon pool would take them). */
void orc_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* ── scalar conversions ─────────────────────────────────────────────────────────────── */

static inline uint32_t f32_bits(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    return u;
}
static inline float bits_f32(uint32_t u) {
    float x;
    memcpy(&x, &u, 4);
    return x;
}

/* bfloat16 from float32, round to nearest even (the `half` crate's bf16::from_f32, which the
 * reference reaches through float32: cast.rs:85-98). */
uint16_t orc_f32_to_bf16(float x) {
    uint32_t u = f32_bits(x);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x0040u);
    uint32_t round_bit = 0x8000u;
    if ((u & round_bit) != 0 && (u & (3 * round_bit - 1)) != 0) return (uint16_t)((u >> 16) + 1);
    return (uint16_t)(u >> 16);
}
float orc_bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

float orc_f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 0x1F, m = h & 0x3FF;
    if (e == 0x1F) return bits_f32(sign | 0x7F800000u | (m << 13));
    if (e == 0) {
        float v = ldexpf((float)m, -24);
        return sign ? -v : v;
    }
    return bits_f32(sign | ((e + 112) << 23) | (m << 13));
}

/* float16 from a double in one rounding to nearest even (the `half` crate's f16::from_f64,
 * cast.rs:70-82). */
uint16_t orc_f64_to_f16(double d) {
    uint16_t sign = signbit(d) ? 0x8000u : 0;
    if (isnan(d)) return sign | 0x7E00u;
    double a = fabs(d);
    if (a >= 65520.0) return sign | 0x7C00u;
    if (a == 0.0) return sign;
    int e;
    (void)frexp(a, &e); /* a = m * 2^e with m in [0.5, 1) */
    int exp = e - 1;
    if (exp < -14) exp = -14;
    double q = ldexp(a, 10 - exp);
    double r = nearbyint(q); /* default rounding mode: ties to even */
    int32_t mant = (int32_t)r;
    int32_t bits = ((exp + 15) << 10) + mant - 1024;
    return sign | (uint16_t)bits;
}

/* Loads element i of a float array of `dtype` as float32 (exact widening). */
static inline float load_f32(const void *p, size_t i, int dtype) {
    switch (dtype) {
    case ORC_F32: return ((const float *)p)[i];
    case ORC_F16: return orc_f16_to_f32(((const uint16_t *)p)[i]);
    default: return orc_bf16_to_f32(((const uint16_t *)p)[i]);
    }
}

/* round_to::<T>(x) for an f64 x (kernels.rs:767-770 with the Scalar impls of cast.rs). */
static inline void store_round(void *p, size_t i, int dtype, double x) {
    switch (dtype) {
    case ORC_F32: ((float *)p)[i] = (float)x; break;
    case ORC_F16: ((uint16_t *)p)[i] = orc_f64_to_f16(x); break;
    default: ((uint16_t *)p)[i] = orc_f32_to_bf16((float)x); break;
    }
}

static size_t dtype_size(int dtype) { return dtype == ORC_F32 ? 4 : 2; }

/* ── fp codecs (fp8.rs) ─────────────────────────────────────────────────────────────── */

#define E4M3_MAX 448.0f
#define E2M1_MAX 6.0f

/* fp8.rs:18-36 */
uint8_t orc_e4m3_from_f32(float x) {
    const uint32_t FP8_MAX = 543u << 21, DENORM_MASK = 141u << 23;
    uint32_t bits = f32_bits(x);
    uint32_t sign = bits & 0x80000000u;
    bits ^= sign;
    uint8_t code;
    if (bits >= FP8_MAX) {
        code = 0x7E;
    } else if (bits < (121u << 23)) {
        float sum = bits_f32(bits) + bits_f32(DENORM_MASK);
        code = (uint8_t)(f32_bits(sum) - DENORM_MASK);
    } else {
        uint32_t odd = (bits >> 20) & 1;
        bits += ((uint32_t)(7 - 127) << 23) + 0x7FFFFu;
        bits += odd;
        code = (uint8_t)(bits >> 20);
    }
    return code | (uint8_t)(sign >> 24);
}

/* fp8.rs:39-44: through float16, times 256, rounded back to float16. */
float orc_e4m3_to_f32(uint8_t code) {
    uint16_t v = code & 127;
    uint16_t sign = (uint16_t)(code >> 7) << 15;
    uint16_t u = (uint16_t)((v << 7) | (((v + 1) >> 7) << 14) | sign);
    float wide = orc_f16_to_f32(u) * 256.0f;
    return orc_f16_to_f32(orc_f64_to_f16((double)wide));
}

/* fp8.rs:48-73 */
uint8_t orc_e2m1_from_f32(float x) {
    if (isnan(x)) return 0x7;
    uint8_t sign = signbit(x) ? 0x8 : 0x0;
    float a = fabsf(x);
    uint8_t code = a > 5.0f ? 7 : a >= 3.5f ? 6 : a > 2.5f ? 5 : a >= 1.75f ? 4
                 : a > 1.25f ? 3 : a >= 0.75f ? 2 : a > 0.25f ? 1 : 0;
    return code | sign;
}

/* fp8.rs:76-80 */
float orc_e2m1_to_f32(uint8_t code) {
    static const float values[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
    float m = values[code & 7];
    return (code & 8) ? -m : m;
}

/* fp8.rs:84-93 */
uint8_t orc_e8m0_from_f32(float x) {
    if (!isfinite(x)) return 0xFF;
    if (x < 0.0f) return 0x00;
    float l = roundf(log2f(x)); /* halves away from zero, as f32::round */
    int n = l <= -127.0f ? -127 : l >= 127.0f ? 127 : (int)l;
    return (uint8_t)(n + 127);
}

/* fp8.rs:96-102 */
float orc_e8m0_to_f32(uint8_t code) {
    return code == 0 ? bits_f32(0x400000u) : bits_f32((uint32_t)code << 23);
}

/* fp8.rs:107-113 */
static inline float ftz(float x) {
    return fpclassify(x) == FP_SUBNORMAL ? copysignf(0.0f, x) : x;
}
/* f32::max / f32::min: a NaN operand of either kind is ignored.  (The C library's fmaxf and fminf
 * return NaN for a SIGNALLING NaN operand, which Rust's do not, so they are spelled out.) */
static inline float max_f32(float a, float b) { return b != b ? a : a != a ? b : (a > b ? a : b); }
static inline float min_f32(float a, float b) { return b != b ? a : a != a ? b : (a < b ? a : b); }
/* fp8.rs:117-119 */
static inline float canonical(float x) { return isnan(x) ? bits_f32(0x7FC00000u) : x; }

/* fp8.rs:124-130 */
float orc_mx_scale_round_up(float x) {
    uint8_t code = orc_e8m0_from_f32(x);
    if (code < 0xFE && ftz(orc_e8m0_to_f32(code)) < x) code += 1;
    return orc_e8m0_to_f32(code);
}

/* ── validation (quantized.rs:137-167) ──────────────────────────────────────────────── */

int orc_check_quant(int mode, int gs, int bits) {
    if (mode == ORC_AFFINE) {
        if (gs != 32 && gs != 64 && gs != 128) return fail("group size %ld is not supported (32, 64 or 128)", gs, 0);
        if (!((bits >= 1 && bits <= 6) || bits == 8)) return fail("%ld bits are not supported (1, 2, 3, 4, 5, 6 or 8)", bits, 0);
        return 0;
    }
    int eg = mode == ORC_NVFP4 ? 16 : 32, eb = mode == ORC_MXFP8 ? 8 : 4;
    if (mode != ORC_MXFP4 && mode != ORC_MXFP8 && mode != ORC_NVFP4) return fail("invalid quantization mode %ld", mode, 0);
    if (gs != eg) return fail("quantization requires group size %ld but got %ld", eg, gs);
    if (bits != eb) return fail("quantization requires bits to be %ld but got %ld", eb, bits);
    return 0;
}

/* ── bit packing (kernels.rs:749-756) ───────────────────────────────────────────────── */

static inline uint32_t code_at(const uint8_t *bytes, size_t i, int bits) {
    size_t byte = i * (size_t)bits / 8, shift = i * (size_t)bits % 8;
    uint32_t v = (uint32_t)bytes[byte] >> shift;
    if (shift + (size_t)bits > 8) v |= (uint32_t)bytes[byte + 1] << (8 - shift);
    return v & ((1u << bits) - 1);
}

/* ── quantize ───────────────────────────────────────────────────────────────────────── */

/* kernels.rs:774-831 */
static void quantize_affine(int gs, int bits, int dtype, const void *w, size_t count,
                            uint32_t *codes, void *scales, void *biases) {
    size_t groups = count / (size_t)gs;
    float n_bins = (float)((1u << bits) - 1);
    const float eps = 1e-7f;
    uint8_t *bytes = (uint8_t *)codes;
    memset(bytes, 0, count * (size_t)bits / 8);
    for (size_t g = 0; g < groups; g++) {
        float lo = INFINITY, hi = -INFINITY;
        for (int j = 0; j < gs; j++) {
            float v = load_f32(w, g * gs + j, dtype);
            lo = min_f32(lo, v); /* f32::min/max ignore a NaN operand */
            hi = max_f32(hi, v);
        }
        float scale, bias;
        if (bits == 1) {
            scale = max_f32(hi - lo, eps);
            bias = lo;
        } else {
            int wide = fabsf(lo) > fabsf(hi);
            scale = max_f32((hi - lo) / n_bins, eps);
            scale = wide ? scale : -scale;
            float edge = wide ? lo : hi;
            float q0 = rintf(edge / scale);
            if (q0 == 0.0f) {
                bias = 0.0f;
            } else {
                scale = edge / q0;
                bias = edge;
            }
        }
        for (int j = 0; j < gs; j++) {
            float v = load_f32(w, g * gs + j, dtype);
            float r = rintf((v - bias) / scale);
            /* f32::clamp keeps NaN; `as u32` maps NaN to 0 */
            r = r < 0.0f ? 0.0f : r > n_bins ? n_bins : r;
            uint32_t q = isnan(r) ? 0u : (uint32_t)r;
            size_t bit = (g * (size_t)gs + j) * (size_t)bits;
            size_t byte = bit / 8, shift = bit % 8;
            uint32_t widev = q << shift;
            bytes[byte] |= (uint8_t)widev;
            if (shift + (size_t)bits > 8) bytes[byte + 1] |= (uint8_t)(widev >> 8);
        }
        store_round(scales, g, dtype, (double)scale);
        store_round(biases, g, dtype, (double)bias);
    }
}

/* kernels.rs:914-971 */
static void quantize_fp(int gs, int bits, int dtype, const void *w, size_t count,
                        const float *global, uint32_t *codes, uint8_t *scale_codes) {
    int mx = gs == 32;
    float max_element = bits == 4 ? E2M1_MAX : E4M3_MAX;
    uint8_t *bytes = (uint8_t *)codes;
    int has_enc = global != NULL;
    float scale_enc = has_enc ? ftz(E4M3_MAX * E2M1_MAX / *global) : 1.0f;
    size_t groups = count / (size_t)gs;
    for (size_t g = 0; g < groups; g++) {
        float amax = 0.0f;
        for (int j = 0; j < gs; j++) amax = max_f32(amax, fabsf(ftz(load_f32(w, g * gs + j, dtype))));
        float scale = ftz(amax / max_element);
        if (has_enc) scale = ftz(scale * scale_enc);
        uint8_t code;
        float decoded;
        if (mx && !has_enc) {
            float rounded = orc_mx_scale_round_up(scale);
            code = orc_e8m0_from_f32(rounded);
            decoded = orc_e8m0_to_f32(code);
        } else {
            code = orc_e4m3_from_f32(scale);
            decoded = orc_e4m3_to_f32(code);
        }
        scale_codes[g] = code;
        decoded = ftz(decoded);
        float inverse = decoded == 0.0f ? 0.0f : ftz((has_enc ? scale_enc : 1.0f) / decoded);
        for (int j = 0; j < gs; j++) {
            size_t i = g * (size_t)gs + j;
            float scaled = canonical(ftz(ftz(load_f32(w, i, dtype)) * inverse));
            if (bits == 8) {
                bytes[i] = orc_e4m3_from_f32(scaled);
            } else {
                uint8_t nibble = orc_e2m1_from_f32(scaled);
                if (i % 2 == 0) bytes[i / 2] = nibble;
                else bytes[i / 2] |= (uint8_t)(nibble << 4);
            }
        }
    }
}

int orc_quantize(int mode, int gs, int bits, int dtype, const void *w, size_t rows, size_t cols,
                 const float *global, uint32_t *codes, void *scales, void *biases) {
    if (orc_check_quant(mode, gs, bits)) return -1;
    if (dtype != ORC_F32 && dtype != ORC_F16 && dtype != ORC_BF16) return fail("quantize: unsupported dtype %ld", dtype, 0);
    if (cols % (size_t)gs != 0) return fail("quantize: last dimension %ld not divisible by the group size %ld", (long)cols, gs);
    if (global && mode != ORC_NVFP4) return fail("quantize: a global scale is only supported for nvfp4", 0, 0);
    if (mode == ORC_AFFINE) quantize_affine(gs, bits, dtype, w, rows * cols, codes, scales, biases);
    else quantize_fp(gs, bits, dtype, w, rows * cols, global, codes, (uint8_t *)scales);
    return 0;
}

/* ── dequantize ─────────────────────────────────────────────────────────────────────── */

/* kernels.rs:835-859: product and sum each rounded to the scales' dtype.  With `fused` the
 * single rounding of the Metal kernel (quantized.h:2701-2705). */
static void dequantize_affine_range(int gs, int bits, int dtype, const uint8_t *bytes,
                                    const void *scales, const void *biases, size_t begin,
                                    size_t end, void *out, int fused) {
    for (size_t i = begin; i < end; i++) {
        size_t g = i / (size_t)gs;
        double c = (double)code_at(bytes, i, bits);
        double s = (double)load_f32(scales, g, dtype), b = (double)load_f32(biases, g, dtype);
        if (fused) {
            store_round(out, i, dtype, (double)fmaf((float)c, (float)s, (float)b));
            continue;
        }
        double product;
        switch (dtype) { /* round_to::<T>(code * scale), then back to f64 */
        case ORC_F32: product = (double)(float)(c * s); break;
        case ORC_F16: product = (double)orc_f16_to_f32(orc_f64_to_f16(c * s)); break;
        default: product = (double)orc_bf16_to_f32(orc_f32_to_bf16((float)(c * s))); break;
        }
        store_round(out, i, dtype, product + b);
    }
}

/* kernels.rs:976-1009 */
static void dequantize_fp_range(int gs, int bits, int dtype, const uint8_t *bytes,
                                const uint8_t *scales, const float *global, size_t begin,
                                size_t end, void *out) {
    int mx = gs == 32;
    int has = global != NULL;
    float inv = has ? ftz(*global / (E4M3_MAX * E2M1_MAX)) : 1.0f;
    for (size_t i = begin; i < end; i++) {
        uint8_t code = scales[i / (size_t)gs];
        float scale = ftz(mx ? orc_e8m0_to_f32(code) : orc_e4m3_to_f32(code));
        if (has) scale = ftz(scale * inv);
        float value = bits == 8 ? orc_e4m3_to_f32(bytes[i])
                                : orc_e2m1_to_f32((bytes[i / 2] >> (4 * (i % 2))) & 0xF);
        store_round(out, i, dtype, (double)canonical(ftz(scale * value)));
    }
}

static void dequantize_any(int mode, int gs, int bits, int dtype, const uint32_t *codes,
                           const void *scales, const void *biases, const float *global,
                           size_t count, void *out, int fused, int parallel) {
    const uint8_t *bytes = (const uint8_t *)codes;
    if (!parallel) {
        if (mode == ORC_AFFINE) dequantize_affine_range(gs, bits, dtype, bytes, scales, biases, 0, count, out, fused);
        else dequantize_fp_range(gs, bits, dtype, bytes, (const uint8_t *)scales, global, 0, count, out);
        return;
    }
    /* Chunks are multiples of 128 values, so no two threads share a group or a byte. */
    size_t chunk = 1 << 14;
    long chunks = (long)((count + chunk - 1) / chunk);
#pragma omp parallel for schedule(static)
    for (long c = 0; c < chunks; c++) {
        size_t b = (size_t)c * chunk, e = b + chunk < count ? b + chunk : count;
        if (mode == ORC_AFFINE) dequantize_affine_range(gs, bits, dtype, bytes, scales, biases, b, e, out, fused);
        else dequantize_fp_range(gs, bits, dtype, bytes, (const uint8_t *)scales, global, b, e, out);
    }
}

int orc_dequantize(int mode, int gs, int bits, int dtype, const uint32_t *codes,
                   const void *scales, const void *biases, const float *global, size_t rows,
                   size_t cols, void *out, int fused) {
    if (orc_check_quant(mode, gs, bits)) return -1;
    if (dtype != ORC_F32 && dtype != ORC_F16 && dtype != ORC_BF16) return fail("dequantize: unsupported dtype %ld", dtype, 0);
    if (mode == ORC_AFFINE && !biases) return fail("dequantize: biases must be provided for affine quantization", 0, 0);
    if (mode != ORC_AFFINE && biases) return fail("dequantize: biases must be null for this mode", 0, 0);
    if (global && mode != ORC_NVFP4) return fail("dequantize: a global scale is only supported for nvfp4", 0, 0);
    if (cols % (size_t)gs != 0) return fail("dequantize: %ld columns not divisible by the group size %ld", (long)cols, gs);
    dequantize_any(mode, gs, bits, dtype, codes, scales, biases, global, rows * cols, out, fused, 0);
    return 0;
}

/* ── sorted_offsets (kernels.rs:875-892) ────────────────────────────────────────────── */

int orc_sorted_offsets(const uint32_t *idx, size_t rows, size_t groups, int32_t *out) {
    for (size_t g = 0; g < groups; g++) {
        size_t lo = 0, hi = rows; /* partition_point(|i| i < g) */
        while (lo < hi) {
            size_t mid = lo + (hi - lo) / 2;
            if ((size_t)idx[mid] < g) lo = mid + 1;
            else hi = mid;
        }
        out[g] = (int32_t)lo;
    }
    return 0;
}

/* ── f32 products (nuvec-cpu) ───────────────────────────────────────────────────────── */

/* few_rows.rs:25-61,133-224: term p goes to partial p mod 8, each partial is a chain of fused
 * multiply-adds from +0 in increasing p, and the partials are combined by one fixed tree. */
static inline float few_rows_dot(const float *x, const float *w, size_t k) {
    float s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    size_t full = k / 8 * 8;
    for (size_t q = 0; q < full; q += 8)
        for (int l = 0; l < 8; l++) s[l] = fmaf(x[q + l], w[q + l], s[l]);
    for (size_t p = full; p < k; p++) s[p - full] = fmaf(x[p], w[p], s[p - full]);
    return ((s[0] + s[4]) + (s[2] + s[6])) + ((s[1] + s[5]) + (s[3] + s[7]));
}

typedef float v8f __attribute__((vector_size(32), aligned(4)));

/* Stand-in for the `gemm` crate (matmul.rs:131-151) above 16 rows: 4 x 2 register tiles of
 * 8-lane partial sums along K.  Its summation order is this file's own. */
static void gemm_nt_block(const float *x, const float *w, size_t M, size_t N, size_t K,
                          float *y, size_t n0, size_t n1) {
    size_t kv = K / 8 * 8;
    for (size_t m0 = 0; m0 < M; m0 += 4) {
        size_t mr = M - m0 < 4 ? M - m0 : 4;
        for (size_t n = n0; n < n1; n += 2) {
            size_t nr = n1 - n < 2 ? n1 - n : 2;
            v8f acc[4][2];
            memset(acc, 0, sizeof acc);
            const float *xr[4], *wr[2];
            for (size_t i = 0; i < 4; i++) xr[i] = x + (m0 + (i < mr ? i : 0)) * K;
            for (size_t j = 0; j < 2; j++) wr[j] = w + (n + (j < nr ? j : 0)) * K;
            for (size_t k = 0; k < kv; k += 8) {
                v8f b0 = *(const v8f *)(wr[0] + k), b1 = *(const v8f *)(wr[1] + k);
                for (int i = 0; i < 4; i++) {
                    v8f a = *(const v8f *)(xr[i] + k);
                    acc[i][0] += a * b0;
                    acc[i][1] += a * b1;
                }
            }
            for (size_t i = 0; i < mr; i++)
                for (size_t j = 0; j < nr; j++) {
                    float s = 0.0f;
                    for (int l = 0; l < 8; l++) s += acc[i][j][l];
                    for (size_t k = kv; k < K; k++) s += xr[i][k] * wr[j][k];
                    y[(m0 + i) * N + n + j] = s;
                }
        }
    }
}

void orc_matmul_nt_f32(const float *x, const float *w, size_t M, size_t N, size_t K, float *y) {
    if (M == 0 || N == 0) return;
    if (K == 0) {
        memset(y, 0, M * N * sizeof(float));
        return;
    }
    if (M <= 16) {
        /* few_rows.rs:84,116-126: parallel over blocks of 64 columns when n*k >= 2^16. */
        long blocks = (long)((N + 63) / 64);
        int parallel = N * K >= ((size_t)1 << 16);
#pragma omp parallel for schedule(static) if (parallel)
        for (long c = 0; c < blocks; c++) {
            size_t j1 = (size_t)(c + 1) * 64 < N ? (size_t)(c + 1) * 64 : N;
            for (size_t j = (size_t)c * 64; j < j1; j++)
                for (size_t i = 0; i < M; i++) y[i * N + j] = few_rows_dot(x + i * K, w + j * K, K);
        }
        return;
    }
    long blocks = (long)((N + 31) / 32);
#pragma omp parallel for schedule(dynamic)
    for (long c = 0; c < blocks; c++) {
        size_t n1 = (size_t)(c + 1) * 32 < N ? (size_t)(c + 1) * 32 : N;
        gemm_nt_block(x, w, M, N, K, y, (size_t)c * 32, n1);
    }
}

static float *widen(const void *p, size_t count, int dtype) {
    float *out = (float *)malloc((count ? count : 1) * sizeof(float));
    if (!out) return NULL;
    for (size_t i = 0; i < count; i++) out[i] = load_f32(p, i, dtype);
    return out;
}

/* The dense f32 matrix the product multiplies by, as [N, K] rows (transposing when the codes
 * are stored [K, N]).  Affine: dequantized in the scales' dtype, then widened (kernels.rs:
 * 1099,716-718); fp modes: decoded straight to f32 (kernels.rs:1100-1105). */
static float *dense_nk(int mode, int gs, int bits, int dtype, int transpose, const uint32_t *w,
                       const void *scales, const void *biases, const float *global, size_t N,
                       size_t K, int parallel) {
    size_t count = N * K;
    float *dense = (float *)malloc((count ? count : 1) * sizeof(float));
    if (!dense) return NULL;
    if (mode == ORC_AFFINE) {
        void *typed = malloc((count ? count : 1) * dtype_size(dtype));
        if (!typed) {
            free(dense);
            return NULL;
        }
        dequantize_any(mode, gs, bits, dtype, w, scales, biases, NULL, count, typed, 0, parallel);
        for (size_t i = 0; i < count; i++) dense[i] = load_f32(typed, i, dtype);
        free(typed);
    } else {
        dequantize_any(mode, gs, bits, ORC_F32, w, scales, NULL, global, count, dense, 0, parallel);
    }
    if (!transpose) { /* stored [K, N] -> [N, K] */
        float *t = (float *)malloc((count ? count : 1) * sizeof(float));
        if (!t) {
            free(dense);
            return NULL;
        }
        for (size_t k = 0; k < K; k++)
            for (size_t n = 0; n < N; n++) t[n * K + k] = dense[k * N + n];
        free(dense);
        dense = t;
    }
    return dense;
}

static int check_product(const char *op, int mode, int gs, int bits, int dtype, int transpose,
                         const void *biases, const float *global, size_t N, size_t K) {
    (void)op;
    if (orc_check_quant(mode, gs, bits)) return -1;
    if (dtype != ORC_F32 && dtype != ORC_F16 && dtype != ORC_BF16) return fail("unsupported dtype %ld", dtype, 0);
    if (mode == ORC_AFFINE && !biases) return fail("biases must be provided for affine quantization", 0, 0);
    if (mode != ORC_AFFINE && biases) return fail("biases must be null for this quantization mode", 0, 0);
    if (global && mode != ORC_NVFP4) return fail("a global scale is only supported for nvfp4", 0, 0);
    size_t cols = transpose ? K : N;
    if (cols % (size_t)gs != 0) return fail("%ld columns not divisible by the group size %ld", (long)cols, gs);
    return 0;
}

/* kernels.rs:1091-1142 */
int orc_quantized_matmul(int mode, int gs, int bits, int dtype, int transpose, const void *x,
                         const uint32_t *w, const void *scales, const void *biases,
                         const float *global, size_t M, size_t N, size_t K, void *y, int flags) {
    if (check_product("quantized_matmul", mode, gs, bits, dtype, transpose, biases, global, N, K)) return -1;
    if (M == 0 || N == 0) return 0;
    float *dense = dense_nk(mode, gs, bits, dtype, transpose, w, scales, biases, global, N, K, flags & 1);
    float *x32 = widen(x, M * K, dtype);
    float *out = (float *)malloc(M * N * sizeof(float));
    if (!dense || !x32 || !out) {
        free(dense), free(x32), free(out);
        return fail("out of memory", 0, 0);
    }
    orc_matmul_nt_f32(x32, dense, M, N, K, out);
    for (size_t i = 0; i < M * N; i++) store_round(y, i, dtype, (double)out[i]);
    free(dense), free(x32), free(out);
    return 0;
}

/* quantized.rs:679-719.  Each expert is decoded once and reused by its batches; the values
 * are the ones the reference recomputes per batch. */
int orc_gather_qmm(int mode, int gs, int bits, int dtype, int transpose, const void *x,
                   const uint32_t *w, const void *scales, const void *biases,
                   const float *global, const uint32_t *lhs, const uint32_t *rhs,
                   size_t batches, size_t M, size_t N, size_t K, size_t experts, void *y,
                   int flags) {
    if (check_product("gather_qmm", mode, gs, bits, dtype, transpose, biases, global, N, K)) return -1;
    if (batches == 0 || M == 0 || N == 0) return 0;
    size_t groups_per = N * K / (size_t)gs, words_per = N * K * (size_t)bits / 32;
    size_t ssz = mode == ORC_AFFINE ? dtype_size(dtype) : 1;
    float **dense = (float **)calloc(experts ? experts : 1, sizeof(float *));
    if (!dense) return fail("out of memory", 0, 0);
    int rc = 0;
    for (size_t b = 0; b < batches && !rc; b++) {
        size_t e = rhs[b];
        if (e >= experts) rc = fail("gather_qmm: index %ld out of range for %ld experts", (long)e, (long)experts);
    }
    for (size_t b = 0; b < batches && !rc; b++) {
        size_t e = rhs[b];
        if (dense[e]) continue;
        /* With a per-expert global scale: decoded f32 weights times gs / (448 * 6)
         * (quantized.rs:697-718), not the scalar path of fp_dequantize. */
        dense[e] = dense_nk(mode, gs, bits, dtype, transpose, w + e * words_per,
                            (const char *)scales + e * groups_per * ssz,
                            biases ? (const char *)biases + e * groups_per * ssz : NULL, NULL,
                            N, K, flags & 1);
        if (!dense[e]) {
            rc = fail("out of memory", 0, 0);
            break;
        }
        if (global) {
            float factor = global[e] / (E4M3_MAX * E2M1_MAX);
            for (size_t i = 0; i < N * K; i++) dense[e][i] = dense[e][i] * factor;
        }
    }
    float *x32 = NULL, *out = NULL;
    if (!rc) {
        out = (float *)malloc(M * N * sizeof(float));
        x32 = (float *)malloc(M * K * sizeof(float));
        if (!out || !x32) rc = fail("out of memory", 0, 0);
    }
    for (size_t b = 0; b < batches && !rc; b++) {
        size_t l = lhs[b];
        for (size_t i = 0; i < M * K; i++) x32[i] = load_f32(x, l * M * K + i, dtype);
        orc_matmul_nt_f32(x32, dense[rhs[b]], M, N, K, out);
        for (size_t i = 0; i < M * N; i++) store_round(y, b * M * N + i, dtype, (double)out[i]);
    }
    for (size_t e = 0; e < experts; e++) free(dense[e]);
    free(dense), free(x32), free(out);
    return rc;
}

/* ── mixture-of-experts glue (fast/imp.rs:2652-2672, 2731-2747; the compositions they stand for:
 *    fast/imp.rs:1586-1600) ────────────────────────────────────────────────────────────────
 *
 * moe_route = argpartition(e - k) -> the last k indices (kernels.rs:231-273: the CPU argpartition
 * is a stable ascending argsort, NaN last), the probabilities at those indices, and with
 * `normalize` those divided by their sum: the sum in float64 over 8 lanes combined by a fixed tree
 * (kernels.rs:609-621, 626-645), rounded to the array's type, then an element-wise divide in that
 * type (f16 / bf16 divide in float32 and round, kernels.rs:1581). */

static int route_less(float x, float y) {
    int xn = x != x, yn = y != y;
    if (!xn && !yn) return x < y;
    return !xn && yn;
}

static double lane_sum(const float *xs, size_t n) {
    double acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (size_t i = 0; i < n; i++) acc[i % 8] += (double)xs[i];
    return ((acc[0] + acc[4]) + (acc[1] + acc[5])) + ((acc[2] + acc[6]) + (acc[3] + acc[7]));
}

int orc_moe_route(int dtype, const void *probs, size_t rows, size_t experts, size_t k, int normalize,
                  uint32_t *out_indices, void *out_scores) {
    if (k < 1 || k > experts) return fail("moe_route: k = %ld must be in 1..=%ld", (long)k, (long)experts);
    float *p = (float *)malloc(sizeof(float) * (experts + k));
    uint32_t *order = (uint32_t *)malloc(sizeof(uint32_t) * experts);
    if (!p || !order) return fail("moe_route: out of memory (%ld experts, %ld)", (long)experts, 0);
    float *top = p + experts;
    for (size_t r = 0; r < rows; r++) {
        for (size_t e = 0; e < experts; e++) p[e] = load_f32(probs, r * experts + e, dtype);
        /* stable ascending order: position of e = number of experts sorting before it */
        for (size_t e = 0; e < experts; e++) {
            size_t rank = 0;
            for (size_t j = 0; j < experts; j++)
                rank += (route_less(p[j], p[e]) || (!route_less(p[e], p[j]) && j < e)) ? 1 : 0;
            order[rank] = (uint32_t)e;
        }
        for (size_t j = 0; j < k; j++) {
            out_indices[r * k + j] = order[experts - k + j];
            top[j] = p[order[experts - k + j]];
        }
        if (normalize) {
            float total;
            { /* the sum, rounded to the array's type */
                uint32_t cell[1];
                store_round(cell, 0, dtype, 0.0 + lane_sum(top, k));
                total = load_f32(cell, 0, dtype);
            }
            for (size_t j = 0; j < k; j++) {
                float q = top[j] / total;
                store_round(out_scores, r * k + j, dtype, (double)q);
            }
        } else {
            for (size_t j = 0; j < k; j++) store_round(out_scores, r * k + j, dtype, (double)top[j]);
        }
    }
    free(p);
    free(order);
    return 0;
}

/* weighted_sum = sum(x * w[..., None], -2): the element-wise product rounded to the array's type
 * (kernels.rs:1191-1195: f16 / bf16 multiply in float32 and round), summed over the k axis in
 * float64 in order and rounded once (kernels.rs:626-645; the reduced axis is not the innermost
 * one, so the sum is element by element). */
int orc_weighted_sum(int dtype, const void *x, const void *w, size_t rows, size_t k, size_t d, void *out) {
    for (size_t r = 0; r < rows; r++)
        for (size_t c = 0; c < d; c++) {
            double s = 0.0;
            for (size_t j = 0; j < k; j++) {
                float prod = load_f32(x, (r * k + j) * d + c, dtype) * load_f32(w, r * k + j, dtype);
                uint32_t cell[1];
                store_round(cell, 0, dtype, (double)prod);
                s += (double)load_f32(cell, 0, dtype);
            }
            store_round(out, r * d + c, dtype, s);
        }
    return 0;
}

/* SwitchProjection::forward's bias (crates/nuvec-lm/src/model.rs:2139-2143): y + bias.take(indices, 0), in
 * place.  Element-wise add in the array's type (kernels.rs:1191-1195: f16 / bf16 add in float32 and
 * round); `take` clamps an index past the end to the last row (kernels.rs:120-133). */
int orc_expert_bias_add(int dtype, void *y, const void *bias, const uint32_t *indices, size_t rows, size_t n, size_t experts) {
    if (rows * n == 0) return 0;
    if (experts == 0) return -1;
    for (size_t r = 0; r < rows; r++) {
        size_t e = indices[r] < experts ? indices[r] : experts - 1;
        for (size_t c = 0; c < n; c++) {
            float sum = load_f32(y, r * n + c, dtype) + load_f32(bias, e * n + c, dtype);
            store_round(y, r * n + c, dtype, (double)sum);
        }
    }
    return 0;
}

/* The bookkeeping of SwitchGlu::forward (crates/nuvec-lm/src/model.rs:2199-2210): order = argsort(flat)
 * (stable, ascending: kernels.rs:231-266), restore = argsort(order), tokens = (pair / k).take(order),
 * sorted = flat.take(order), offsets = sorted_offsets(sorted) (kernels.rs:875-892).  Plain insertion of
 * every pair behind the pairs of smaller or equal experts that came before it. */
int orc_moe_sort(const uint32_t *indices, size_t pairs, size_t k, size_t experts, uint32_t *order, uint32_t *restore,
                 uint32_t *tokens, uint32_t *sorted, int32_t *offsets) {
    if (k == 0) return -1;
    size_t *next = (size_t *)calloc(experts + 1, sizeof(size_t));
    if (!next) return -1;
    for (size_t i = 0; i < pairs; i++) {
        if (indices[i] >= experts) { free(next); return -1; }
        next[indices[i] + 1]++;
    }
    for (size_t e = 0; e < experts; e++) next[e + 1] += next[e];
    for (size_t e = 0; e < experts; e++) offsets[e] = (int32_t)next[e];
    for (size_t i = 0; i < pairs; i++) {
        size_t pos = next[indices[i]]++;
        order[pos] = (uint32_t)i;
        restore[i] = (uint32_t)pos;
        tokens[pos] = (uint32_t)(i / k);
        sorted[pos] = indices[i];
    }
    free(next);
    return 0;
}

/* MLX's Sigmoid as the reference computes it (crates/nuvec-core/src/kernels.rs:1538-1543), float32. */
static float sigmoid_f32(float x) {
    volatile float a = x < 0.0f ? -x : x;
    volatile float e = expf(a);
    volatile float d = 1.0f + e;
    volatile float y = 1.0f / d;
    return x < 0.0f ? y : 1.0f - y;
}
static float round_to(float v, int dtype) {
    uint32_t cell[1];
    store_round(cell, 0, dtype, (double)v);
    return load_f32(cell, 0, dtype);
}
static float min_nan(float a, float b) { return (a != a || b != b) ? NAN : (a < b ? a : b); }
static float max_nan(float a, float b) { return (a != a || b != b) ? NAN : (a > b ? a : b); }

/* nuvec_nn::swiglu / swiglu_oai (crates/nuvec-nn/src/lib.rs:513-579) as the CPU evaluates the compiled
 * function: its operations one by one (crates/nuvec-core/src/fused.rs:214-217), each rounded to the array's
 * type (kernels.rs:1576-1590: f16 / bf16 compute in float32 and round); alpha and limit are weak scalars,
 * rounded to the type first (lib.rs:504-507).  oai = 0: silu(gate) * up = (gate * sigmoid(gate)) * up. */
int orc_swiglu(int dtype, int oai, const void *gate, const void *up, float alpha, float limit, size_t n, void *out) {
    alpha = round_to(alpha, dtype);
    limit = round_to(limit, dtype);
    for (size_t i = 0; i < n; i++) {
        float g = load_f32(gate, i, dtype), x = load_f32(up, i, dtype);
        volatile float r;
        if (oai) {
            g = min_nan(g, limit);
            x = min_nan(max_nan(x, -limit), limit);
            volatile float ag = alpha * g;
            float s = round_to(sigmoid_f32(round_to(ag, dtype)), dtype);
            volatile float gs0 = g * s;
            float gs = round_to(gs0, dtype);
            volatile float x1 = x + 1.0f;
            r = round_to(x1, dtype) * gs;
        } else {
            float s = round_to(sigmoid_f32(g), dtype);
            volatile float t0 = g * s;
            r = round_to(t0, dtype) * x;
        }
        store_round(out, i, dtype, (double)r);
    }
    return 0;
}

/* fast::rms_norm / fast::add_rms_norm as their CPU expansion computes them
 * (crates/nuvec-core/src/fast/imp.rs:1367-1379 over ops/imp.rs:546-555 and kernels.rs:611-645, 1418):
 *   xf = float32(x) (x + residual first, rounded to the array's type, for add_rms_norm);
 *   s  = float32(lane_sum(xf * xf))        -- float64 over 8 lanes, fixed tree;
 *   n  = 1 / sqrt(s * float32(1 / d) + eps)  -- float32 throughout;
 *   y  = T(xf * n), then T(y * weight) when there is a weight.
 * residual, weight and sum_out may be NULL. */
int orc_rms_norm(int dtype, const void *x, const void *residual, const void *weight, float eps, size_t rows, size_t d, void *sum_out,
                 void *y) {
    float *xf = (float *)malloc((d ? d : 1) * sizeof(float));
    if (!xf) return -1;
    volatile float inv_count = (float)(1.0 / (double)d);
    for (size_t r = 0; r < rows; r++) {
        double acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (size_t j = 0; j < d; j++) {
            float v = load_f32(x, r * d + j, dtype);
            if (residual) {
                volatile float h = v + load_f32(residual, r * d + j, dtype);
                v = round_to(h, dtype);
                if (sum_out) store_round(sum_out, r * d + j, dtype, (double)v);
            }
            xf[j] = v;
        }
        size_t whole = d / 8 * 8;
        for (size_t j = 0; j < whole; j += 8)
            for (size_t l = 0; l < 8; l++) {
                volatile float sq = xf[j + l] * xf[j + l];
                acc[l] += (double)sq;
            }
        for (size_t l = 0; l < d - whole; l++) {
            volatile float sq = xf[whole + l] * xf[whole + l];
            acc[l] += (double)sq;
        }
        volatile double total = ((acc[0] + acc[4]) + (acc[1] + acc[5])) + ((acc[2] + acc[6]) + (acc[3] + acc[7]));
        volatile float s = (float)total;
        volatile float mean = s * inv_count;
        volatile float v = mean + eps;
        volatile float root = sqrtf(v);
        volatile float n = 1.0f / root;
        for (size_t j = 0; j < d; j++) {
            volatile float scaled = xf[j] * n;
            float out = round_to(scaled, dtype);
            if (weight) {
                volatile float ww = out * load_f32(weight, j, dtype);
                out = round_to(ww, dtype);
            }
            store_round(y, r * d + j, dtype, (double)out);
        }
    }
    free(xf);
    return 0;
}
