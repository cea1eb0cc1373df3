// Few-row quantized products (decode): y[m, n] = sum_k x[m, k] * dequantize(w)[n, k].
//
// Two kernels:
//
//  * qmv_affine_kernel -- the fast path for affine 2/4/8-bit weights and up to 8 rows of
//    bfloat16 activations.  It is bound by HBM: the packed words are read once with
//    coalesced vector loads (no L1 allocation), unpacked in registers and accumulated in
//    float32.  At 4 bits the memory system delivers a weight every ~0.3 issue slots per lane,
//    so the multiply-accumulate cannot be afforded on the FMA pipe; the unpacked codes are
//    fed to the warp-level tensor-core MMA (m16n8k16, bf16 in, f32 accumulate) instead, used
//    here purely as a wide dot-product unit: a warp multiplies 16 weight rows x 16 k-values
//    by up to 8 activation rows per instruction.  Every weight is rebuilt in registers with the
//    reference's own two bfloat16 roundings (packed fma/add), so the operands of the product
//    are bit-identical to the reference's dequantized matrix; only the float32 summation order
//    differs.
//
//  * qmv_generic_kernel -- every other case (all bit widths and modes, f32/f16/bf16, any
//    K, both weight orientations).  It rebuilds each weight with exactly the reference's
//    roundings (crates/nuvec-core/src/kernels.rs:835-859, 976-1009) and accumulates in f32.
//
// Reference behaviour covered: MLX/nuvec's qmv, qmv_fast, qmv_wide, qmv_rows and qvm kernels
// (crates/nuvec-kernels/src/metal/quantized.h:819-1342, routing crates/nuvec-core/src/gpu.rs:
// 6934-7168); CPU result crates/nuvec-core/src/kernels.rs:1091-1142.
#include "qmv.cuh"

namespace nvc {

// ── generic kernels ────────────────────────────────────────────────────────────────────

template <typename T>
__device__ __forceinline__ float decode_weight(const GenericParams &p, const uint8_t *wbytes, const void *scales,
                                               const void *biases, size_t idx, float fp_scale_mul) {
    // idx: flat index of the value inside this matrix (row-major, `cols` values per row).
    size_t g = idx / (size_t)p.gs;
    if (p.mode == NVC_AFFINE) {
        float c = (float)code_at(wbytes, idx, p.bits);
        float s = DT<T>::load((const T *)scales, g), b = DT<T>::load((const T *)biases, g);
        float prod = DT<T>::round(__fmul_rn(c, s));
        return DT<T>::round(__fadd_rn(prod, b));
    }
    uint32_t sc = ((const uint8_t *)scales)[g];
    float scale = ftz(p.gs == 32 ? e8m0_to_f32(sc) : e4m3_to_f32(sc));
    if (p.scalar_global) scale = ftz(__fmul_rn(scale, fp_scale_mul));
    float v = p.bits == 8 ? e4m3_to_f32(wbytes[idx]) : e2m1_to_f32((wbytes[idx >> 1] >> (4 * (idx & 1))) & 0xFu);
    float w = canonical(ftz(__fmul_rn(scale, v)));
    if (p.expert_global) w = __fmul_rn(w, fp_scale_mul);
    return w;
}

// One warp per output column (transposed weights): lanes stride over K, up to 8 rows of x per
// pass.  blockIdx.y walks the batch (or the gathered rows).
template <typename T>
__global__ void __launch_bounds__(128) qmv_generic_t_kernel(GenericParams p) {
    const int lane = threadIdx.x & 31;
    const int64_t n = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    const int64_t b = blockIdx.y;
    if (n >= p.N) return;
    int64_t xb = b, wb = b;
    if (p.rhs) {
        wb = p.rhs[b];
        xb = p.lhs ? p.lhs[b] : b;
    }
    const T *x = (const T *)p.x + xb * p.x_batch_stride;
    const uint8_t *w = (const uint8_t *)(p.w + wb * p.w_batch_stride);
    const size_t ssz = p.mode == NVC_AFFINE ? sizeof(T) : 1;
    const char *scales = (const char *)p.scales + wb * p.s_batch_stride * ssz;
    const char *biases = p.biases ? (const char *)p.biases + wb * p.s_batch_stride * ssz : nullptr;
    float mul = 1.0f;
    if (p.scalar_global) mul = ftz(__fdiv_rn(*p.global, 448.0f * 6.0f));
    if (p.expert_global) mul = __fdiv_rn(p.global[wb], 448.0f * 6.0f);
    T *y = (T *)p.y + b * p.M * p.N;
    for (int64_t m0 = 0; m0 < p.M; m0 += 8) {
        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; i++) acc[i] = 0.0f;
        for (int64_t k = lane; k < p.K; k += 32) {
            float wv = decode_weight<T>(p, w, scales, biases, (size_t)(n * p.K + k), mul);
#pragma unroll
            for (int i = 0; i < 8; i++)
                if (m0 + i < p.M) acc[i] = __fmaf_rn(DT<T>::load(x, (size_t)((m0 + i) * p.ldx + k)), wv, acc[i]);
        }
#pragma unroll
        for (int i = 0; i < 8; i++) {
            float v = acc[i];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
            if (lane == 0 && m0 + i < p.M) DT<T>::store(y, (size_t)((m0 + i) * p.N + n), v);
        }
    }
}

// Untransposed weights ([K, N] codes): one thread per output column, K walked serially.
template <typename T>
__global__ void __launch_bounds__(128) qmv_generic_n_kernel(GenericParams p) {
    const int64_t n = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t b = blockIdx.y;
    if (n >= p.N) return;
    int64_t xb = b, wb = b;
    if (p.rhs) {
        wb = p.rhs[b];
        xb = p.lhs ? p.lhs[b] : b;
    }
    const T *x = (const T *)p.x + xb * p.x_batch_stride;
    const uint8_t *w = (const uint8_t *)(p.w + wb * p.w_batch_stride);
    const size_t ssz = p.mode == NVC_AFFINE ? sizeof(T) : 1;
    const char *scales = (const char *)p.scales + wb * p.s_batch_stride * ssz;
    const char *biases = p.biases ? (const char *)p.biases + wb * p.s_batch_stride * ssz : nullptr;
    float mul = 1.0f;
    if (p.scalar_global) mul = ftz(__fdiv_rn(*p.global, 448.0f * 6.0f));
    if (p.expert_global) mul = __fdiv_rn(p.global[wb], 448.0f * 6.0f);
    T *y = (T *)p.y + b * p.M * p.N;
    for (int64_t m0 = 0; m0 < p.M; m0 += 8) {
        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; i++) acc[i] = 0.0f;
        for (int64_t k = 0; k < p.K; k++) {
            float wv = decode_weight<T>(p, w, scales, biases, (size_t)(k * p.N + n), mul);
#pragma unroll
            for (int i = 0; i < 8; i++)
                if (m0 + i < p.M) acc[i] = __fmaf_rn(DT<T>::load(x, (size_t)((m0 + i) * p.ldx + k)), wv, acc[i]);
        }
#pragma unroll
        for (int i = 0; i < 8; i++)
            if (m0 + i < p.M) DT<T>::store(y, (size_t)((m0 + i) * p.N + n), acc[i]);
    }
}

template <typename T> static int32_t launch_generic_typed(nvc_device *dev, const GenericParams &p) {
    if (p.transpose) {
        dim3 grid((unsigned)((p.N + 3) / 4), (unsigned)p.batch);
        qmv_generic_t_kernel<T><<<grid, 128, 0, dev->stream>>>(p);
        return check_launch(dev, "qmv_generic_t_kernel");
    }
    dim3 grid((unsigned)((p.N + 127) / 128), (unsigned)p.batch);
    qmv_generic_n_kernel<T><<<grid, 128, 0, dev->stream>>>(p);
    return check_launch(dev, "qmv_generic_n_kernel");
}

int32_t launch_generic(nvc_device *dev, const GenericParams &p) {
    if (p.batch == 0 || p.M == 0 || p.N == 0) return NVC_OK;
    if (p.batch > 65535) return set_error(NVC_ERR_UNSUPPORTED, "generic product: %lld batches exceed the grid limit", (long long)p.batch);
    switch (p.dtype) {
    case NVC_F32: return launch_generic_typed<float>(dev, p);
    case NVC_F16: return launch_generic_typed<__half>(dev, p);
    default: return launch_generic_typed<__nv_bfloat16>(dev, p);
    }
}

// ── fast affine kernel ─────────────────────────────────────────────────────────────────

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t orv) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;\n" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));  // (a & mask) | orv
    return r;
}
// Packed bfloat16 arithmetic, each lane rounded to nearest even once.
__device__ __forceinline__ uint32_t bf2_fma(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("fma.rn.bf16x2 %0, %1, %2, %3;\n" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}
// a + b as fma(a, 1, b): the same single rounding, and it stays on the FMA pipe (the packed
// bfloat16 add was observed to issue on the quarter-rate conversion pipe).
__device__ __forceinline__ uint32_t bf2_add(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("fma.rn.bf16x2 %0, %1, %2, %3;\n" : "=r"(r) : "r"(a), "r"(0x3F803F80u), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t bf2_mul(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("mul.rn.bf16x2 %0, %1, %2;\n" : "=r"(r) : "r"(a), "r"(b));
    return r;
}

// Asynchronous global -> shared copies of packed words (4, 8 or 16 bytes per lane).  Every lane
// copies into a slot only it reads back, so completion is tracked per thread with
// wait_group and no barrier is involved.  The 16-byte form bypasses L1.
template <int BYTES> __device__ __forceinline__ void cp_async(uint32_t smem_addr, const void *gptr) {
    if (BYTES == 16)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_addr), "l"(gptr) : "memory");
    else if (BYTES == 8)
        asm volatile("cp.async.ca.shared.global [%0], [%1], 8;\n" ::"r"(smem_addr), "l"(gptr) : "memory");
    else
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(smem_addr), "l"(gptr) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

// Per (row, group) constants: {s, s} and {b, b} as bfloat16 pairs staged in shared memory,
// {-128 s, -128 s} derived from them.
struct GroupConsts { uint32_t s2, ns2, b2; };
__device__ __forceinline__ GroupConsts group_consts(uint2 sb) {
    return GroupConsts{sb.x, bf2_mul(sb.x, 0xC300C300u), sb.y};  // -128 * s is exact
}

// Dequantization of one packed word into MMA operands with exactly the reference's two
// roundings (kernels.rs:835-859): p = rn(code * scale), w = rn(p + bias), both in bfloat16.
// A code enters as the bfloat16 number 128 + code (its bits ORed into the mantissa of 128.0);
// fma(128 + c, s, -128 s) is the single rounding of the exact product c * s.
template <int BITS> struct Unpack;
template <> struct Unpack<4> {
    static constexpr int WBITS = 4, FP = 0;
    static constexpr int UW = 1;      // words per unit (the smallest run of words holding whole codes)
    static constexpr int CODES = 8;   // codes per unit
    static constexpr int AREGS = 4;   // operand registers per unit; MMAs per unit = AREGS / 2
    // register i = codes (i, i+4)
    static __device__ __forceinline__ void run(const uint32_t *u, const GroupConsts &c, uint32_t (&r)[4]) {
        const uint32_t w = u[0];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            uint32_t m = lop3_and_or(w >> (4 * i), 0x000F000Fu, 0x43004300u);
            r[i] = bf2_add(bf2_fma(m, c.s2, c.ns2), c.b2);
        }
    }
    // Activation order matching run(): pairs (x0,x4) (x1,x5) (x2,x6) (x3,x7).
    static __device__ __forceinline__ void permute(const uint16_t *x, uint16_t *out) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            out[2 * i] = x[i];
            out[2 * i + 1] = x[i + 4];
        }
    }
};
template <> struct Unpack<8> {
    static constexpr int WBITS = 8, FP = 0;
    static constexpr int UW = 1;
    static constexpr int CODES = 4;
    static constexpr int AREGS = 2;
    // The byte is rebuilt from its nibbles, exactly: 16 * hi + lo <= 255 fits bfloat16.
    // register 0 = codes (0, 2), register 1 = codes (1, 3)
    static __device__ __forceinline__ void run(const uint32_t *u, const GroupConsts &c, uint32_t (&r)[2]) {
        const uint32_t w = u[0];
        const uint32_t k16 = 0x41804180u, kn2048 = 0xC500C500u, kn128 = 0xC300C300u;
#pragma unroll
        for (int i = 0; i < 2; i++) {
            uint32_t lo = lop3_and_or(w >> (8 * i), 0x000F000Fu, 0x43004300u);
            uint32_t hi = lop3_and_or(w >> (8 * i + 4), 0x000F000Fu, 0x43004300u);
            uint32_t code = bf2_add(bf2_fma(hi, k16, kn2048), bf2_add(lo, kn128));  // 16*hi + lo, exact
            r[i] = bf2_add(bf2_mul(code, c.s2), c.b2);
        }
    }
    static __device__ __forceinline__ void permute(const uint16_t *x, uint16_t *out) {
        out[0] = x[0]; out[1] = x[2]; out[2] = x[1]; out[3] = x[3];
    }
};
template <> struct Unpack<2> {
    static constexpr int WBITS = 2, FP = 0;
    static constexpr int UW = 1;
    static constexpr int CODES = 16;
    static constexpr int AREGS = 8;
    // register i = codes (i, i+8)
    static __device__ __forceinline__ void run(const uint32_t *u, const GroupConsts &c, uint32_t (&r)[8]) {
        const uint32_t w = u[0];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            uint32_t m = lop3_and_or(w >> (2 * i), 0x00030003u, 0x43004300u);
            r[i] = bf2_add(bf2_fma(m, c.s2, c.ns2), c.b2);
        }
    }
    static __device__ __forceinline__ void permute(const uint16_t *x, uint16_t *out) {
#pragma unroll
        for (int i = 0; i < 8; i++) {
            out[2 * i] = x[i];
            out[2 * i + 1] = x[i + 8];
        }
    }
};

// 32 bits of a unit's bit stream starting at bit `pos` (a compile-time position once unrolled).
__device__ __forceinline__ uint32_t window3(const uint32_t *u, int pos) {
    const int idx = pos >> 5, sh = pos & 31;
    if (sh == 0) return u[idx];
    if (idx + 1 < 3) return __funnelshift_r(u[idx], u[idx + 1], sh);
    return u[idx] >> sh;
}
// 3 bits: codes straddle words; the unit is 3 words = 32 codes at bit 3c.  Codes 6 apart are 18
// bits apart, so one funnel shift brings code A to bits [2:0] and code A + 6 to bits [20:18] of
// the same register: as bfloat16 mantissas these are 128 + a and 128 + 4 b, and
// fma({128 + a, 128 + 4b}, {s, s/4}, {-128 s, -32 s}) is the single rounding of {a s, b s} (powers
// of two scale exactly).  14 registers are such pairs -- (A, A + 6) for A = 0..5, 12..17, 24, 25 --
// and the four codes left over, 26..29, make two pairs with one extraction per code.
template <> struct Unpack<3> {
    static constexpr int WBITS = 3, FP = 0;
    static constexpr int UW = 3;
    static constexpr int CODES = 32;
    static constexpr int AREGS = 16;
    static __host__ __device__ constexpr int code_a(int i) { return i < 6 ? i : i < 12 ? i + 6 : i < 14 ? i + 12 : i == 14 ? 26 : 28; }
    static __host__ __device__ constexpr int code_b(int i) { return i < 14 ? code_a(i) + 6 : code_a(i) + 1; }
    static __device__ __forceinline__ void run(const uint32_t *u, const GroupConsts &c, uint32_t (&r)[16]) {
        const uint32_t s4 = bf2_mul(c.s2, 0x3E803F80u);   // {s, s / 4}
        const uint32_t ns4 = bf2_mul(s4, 0xC300C300u);    // {-128 s, -32 s}
#pragma unroll
        for (int i = 0; i < 14; i++) {
            const uint32_t m = lop3_and_or(window3(u, 3 * code_a(i)), 0x001C0007u, 0x43004300u);
            r[i] = bf2_add(bf2_fma(m, s4, ns4), c.b2);
        }
#pragma unroll
        for (int i = 14; i < 16; i++) {
            const uint32_t lo = lop3_and_or(window3(u, 3 * code_a(i)), 0x00000007u, 0x43004300u);
            const uint32_t m = lop3_and_or(window3(u, 3 * code_b(i) - 16), 0x00070000u, lo);
            r[i] = bf2_add(bf2_fma(m, c.s2, c.ns2), c.b2);
        }
    }
    static __device__ __forceinline__ void permute(const uint16_t *x, uint16_t *out) {
#pragma unroll
        for (int i = 0; i < 16; i++) {
            out[2 * i] = x[code_a(i)];
            out[2 * i + 1] = x[code_b(i)];
        }
    }
};
// 6 bits: the unit is 3 words = 16 codes at bit 6c; codes up to 63 leave no room to scale the
// upper one, so each code of a pair takes its own extraction.  register i = codes (i, i + 8).
template <> struct Unpack<6> {
    static constexpr int WBITS = 6, FP = 0;
    static constexpr int UW = 3;
    static constexpr int CODES = 16;
    static constexpr int AREGS = 8;
    static __device__ __forceinline__ void run(const uint32_t *u, const GroupConsts &c, uint32_t (&r)[8]) {
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const uint32_t lo = lop3_and_or(window3(u, 6 * i), 0x0000003Fu, 0x43004300u);
            const uint32_t m = lop3_and_or(window3(u, 6 * (i + 8) - 16), 0x003F0000u, lo);
            r[i] = bf2_add(bf2_fma(m, c.s2, c.ns2), c.b2);
        }
    }
    static __device__ __forceinline__ void permute(const uint16_t *x, uint16_t *out) {
#pragma unroll
        for (int i = 0; i < 8; i++) {
            out[2 * i] = x[i];
            out[2 * i + 1] = x[i + 8];
        }
    }
};

// 4-bit floating point (E2M1 codes; kernel "bits" 40 = mxfp4: one E8M0 scale per 32 values,
// 41 = nvfp4: one E4M3 scale per 16).  The code's three magnitude bits become exponent[1:0] and
// mantissa[6] of a bfloat16 whose value is magnitude * 2^-126 (the subnormal codes 0 and 0.5
// included); multiplying by 2^126 restores the value and multiplying by the scale (a power of
// two, or an E4M3 number with 4 significant bits) is exact: at most 6 significant bits.  The
// operand equals the reference's float32 decode (crates/nuvec-core/src/kernels.rs:976-1009).
// register i = codes (i, i+4), as for 4-bit affine.  c.s2 holds the decoded scale pair.
template <int KIND> struct UnpackFp4 {
    static constexpr int WBITS = 4, FP = KIND;
    static constexpr int UW = 1;
    static constexpr int CODES = 8;
    static constexpr int AREGS = 4;
    static __device__ __forceinline__ void run(const uint32_t *u, const GroupConsts &c, uint32_t (&r)[4]) {
        const uint32_t w = u[0];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            // magnitude bits [2:0] of both codes -> bits [8:6] of their halves; sign bit 3 -> bit 15
            const uint32_t mag = 4 * i >= 6 ? (w >> (4 * i - 6)) : (w << (6 - 4 * i));
            const uint32_t sgn = 4 * i >= 12 ? (w >> (4 * i - 12)) : (w << (12 - 4 * i));
            const uint32_t bits = lop3_and_or(sgn, 0x80008000u, mag & 0x01C001C0u);
            r[i] = bf2_mul(bf2_mul(bits, 0x7E807E80u), c.s2);
        }
    }
    static __device__ __forceinline__ void permute(const uint16_t *x, uint16_t *out) { Unpack<4>::permute(x, out); }
};
template <> struct Unpack<40> : UnpackFp4<1> {};
template <> struct Unpack<41> : UnpackFp4<3> {};
// bfloat16 pair {s, s} of a scale code: E8M0 (2^(code - 127); code 0 decodes to a float32 subnormal
// that the reference flushes to zero) or E4M3 (subnormal results flushed likewise).
__device__ __forceinline__ uint32_t fp4_scale2(uint32_t code, bool e8m0) {
    uint32_t h;
    if (e8m0) h = code == 0u ? 0u : (code << 7);
    else h = __float_as_uint(ftz(e4m3_to_f32(code))) >> 16;
    return (h & 0xFFFFu) * 0x10001u;
}

constexpr int QMV_WARPS = 8;
constexpr int QMV_THREADS = QMV_WARPS * 32;
// Resident blocks per multiprocessor the kernel is compiled for (128 registers per thread; three
// blocks at 80 registers were measured slower at every size).
constexpr int QMV_BLOCKS_PER_SM = 2;
// Depth of each lane's ring of asynchronous weight copies (iterations in flight per warp): the
// bytes in flight per lane stay near 128 whatever the iteration's width.
__host__ __device__ constexpr int qmv_stages(int wpl) { return wpl == 8 ? 3 : 4; }
// Most groups whose scale/bias are staged at a time (one k-chunk of a tile).
constexpr int QMV_SEG_GROUPS = 16;
// Row pitch (bfloat16 elements) of the staged scales: 48 bytes = 12 banks, a multiple of 16 bytes
// (the widest copy); the 8 rows a warp reads together fall on different banks.
constexpr int QMV_SPITCH = QMV_SEG_GROUPS + 8;
// 4-bit floating point: up to 64 groups (bytes) of a row per k-chunk, rows 80 bytes apart (20 banks:
// the 8 rows a warp reads together fall on different banks); 2 x 16 x 80 bytes fit the same area.
constexpr int QMV_FP_SEG_GROUPS = 64;
constexpr int QMV_FPITCH = 80;
static_assert(2 * 16 * QMV_FPITCH <= 4 * 16 * QMV_SPITCH * 2, "the floating-point scale buffers fit the per-warp scale area");

// The product is cut into iterations: iteration (tile, i) multiplies 16 weight rows ("tile") by
// IK = 4 * WPL * CODES consecutive k-values.  All iterations of all tiles form one sequence, tile
// after tile, and the warps of the grid take equal consecutive runs of it (stream-K): the load is
// balanced to one iteration whatever N and K are.  A warp that holds a whole tile writes the
// result; tiles cut by a run boundary leave float32 partials in scratch and the warp that
// arrives last adds them in run order.  Warps share the staged activations and nothing else, so
// the main loop has no block-wide barrier.
//
// Lane (r, t) = (lane / 4, lane % 4) holds rows r and r + 8 of the tile and, per iteration, WPL
// consecutive words of each (a quad covers the IK k-values).  The words travel through a per-lane
// ring of cp.async copies that keeps running across tile boundaries, so HBM requests stay in
// flight while a tile is finished and the next one starts.
//
// Shared memory:
//   xs    [M][pitch] u32      all activations in MMA operand order: the chunk of word j of lane t
//                             in iteration i sits at ((i * WPL + j) * 4 + t) * XW
//   zero  [64] u32            what lanes of activation rows >= M read
//   per warp:
//   sraw, braw [2][16][QMV_SPITCH] bf16   scales / biases of the current and the next k-chunk
//   ring  [stages][2][32] x WPL u32       packed words in flight: slot (stage, row half, lane);
//                                         WPL = 8 keeps its two 16-byte chunks 512 bytes apart
//                                         (chunk, lane) so that a quarter-warp reads 128
//                                         consecutive bytes
//   lpart [QMV_WARPS][2][128] f32         partial sums of tiles cut between warps of this block
//   lcount[QMV_WARPS + 4] u32             their arrival counters; word QMV_WARPS: "this block finished last" (fused gather)
template <int BITS, int WPL>
__global__ void __launch_bounds__(QMV_THREADS, QMV_BLOCKS_PER_SM) qmv_affine_kernel(QmvParams p) {
    using U = Unpack<BITS>;
    constexpr int CODES = U::CODES, AREGS = U::AREGS, UW = U::UW;
    constexpr int LW = WPL * UW;               // words per lane, row half and iteration (WPL units of UW words)
    constexpr int IK = 4 * WPL * CODES;
    constexpr int XW = AREGS;  // activation words per unit (AREGS bf16 pairs)
    constexpr int QMV_STAGES = qmv_stages(WPL);
    // copies per lane and row half: 3-word units are only 4-byte aligned and go word by word
    constexpr int CPL = UW == 3 ? LW : WPL == 8 ? 2 : 1;
    constexpr int CW = LW / CPL;               // words per copy
    extern __shared__ __align__(16) uint32_t smem[];

    const int tid = threadIdx.x, lane = tid & 31;
    // the warp index read from lane 0: the compiler then knows that everything derived from it (run
    // bounds, loop trip counts) is the same for the whole warp and keeps mma.sync free of re-convergence code
    const int warp = __shfl_sync(0xFFFFFFFFu, tid >> 5, 0);
    const int r = lane >> 2, t = lane & 3;
    const int64_t b = blockIdx.z;
    int64_t xb = b, wb = b;
    if (p.rhs) {
        wb = p.rhs[b];
        xb = p.lhs ? p.lhs[b] : b;
    }
    const int row_groups = (int)(p.K >> p.gs_shift);
    const uint32_t row_words = (uint32_t)(p.K * U::WBITS / 32);
    const int ipt = (int)(p.K / IK);        // iterations per tile
    const int ci = p.chunk_k / IK;          // iterations per k-chunk (scales are staged per chunk)
    const int chunk_groups = p.chunk_k >> p.gs_shift;
    const int tiles = (int)((p.N + 15) / 16);
    const int last_row = (int)p.N - 1;

    const int xs_pitch = (int)(p.K / CODES) * XW + 16;  // words; = 16 (mod 32) keeps two rows on disjoint banks
    uint32_t *xs = smem;
    uint32_t *zero = xs + (size_t)p.M * xs_pitch;
    uint16_t *sraw = reinterpret_cast<uint16_t *>(zero + 64) + (size_t)warp * (4 * 16 * QMV_SPITCH);
    uint16_t *braw = sraw + 2 * 16 * QMV_SPITCH;
    uint32_t *ring = reinterpret_cast<uint32_t *>(reinterpret_cast<uint16_t *>(zero + 64) +
                                                  (size_t)QMV_WARPS * (4 * 16 * QMV_SPITCH)) +
                     (size_t)warp * (QMV_STAGES * 2 * 32 * LW);
    const uint32_t ring_s = (uint32_t)__cvta_generic_to_shared(ring + lane * CW);
    float *lpart = reinterpret_cast<float *>(ring + (size_t)(QMV_WARPS - warp) * (QMV_STAGES * 2 * 32 * LW));
    uint32_t *lcount = reinterpret_cast<uint32_t *>(lpart + QMV_WARPS * 2 * 128);
    constexpr uint32_t HALF_BYTES = 32 * LW * 4, STAGE_BYTES = 2 * HALF_BYTES;

    // ── this warp's run of iterations ───────────────────────────────────────────────────
    // Two levels: the blocks take consecutive runs of the sequence whose lengths differ by at most
    // one (the first blk_r blocks hold blk_q + 1 iterations) and the warps of a block split the
    // block's run the same way.  The launch gives every block at least QMV_WARPS iterations unless
    // the grid is a single block, where surplus warps idle.  All of it is 32-bit arithmetic: the
    // launch refuses sequences of 2^30 iterations or more.
    const uint32_t blk_q = p.blk_q, blk_r = p.blk_r;
    // Run of part `i` when `len`-sized work is cut into parts of q or q + 1 (the first rm parts).
    auto part_lo = [](uint32_t i, uint32_t q, uint32_t rm) { return i * q + min(i, rm); };
    auto part_of = [](uint32_t at, uint32_t q, uint32_t rm) {
        const uint32_t big = rm * (q + 1u);
        return at < big ? at / (q + 1u) : rm + (at - big) / q;
    };
    const uint32_t blk_lo = part_lo(blockIdx.x, blk_q, blk_r), blk_len = blk_q + (blockIdx.x < blk_r ? 1u : 0u);
    const uint32_t nw = min((uint32_t)QMV_WARPS, blk_len);
    const uint32_t wq = nw == QMV_WARPS ? blk_len / QMV_WARPS : 1u, wr = nw == QMV_WARPS ? blk_len % QMV_WARPS : 0u;
    const uint32_t lo = (uint32_t)warp < nw ? blk_lo + part_lo(warp, wq, wr) : 0u;
    const uint32_t hi = (uint32_t)warp < nw ? lo + wq + ((uint32_t)warp < wr ? 1u : 0u) : 0u;
    // Block and warp whose run holds iteration i.
    auto owner = [&](uint32_t i, uint32_t &cta, uint32_t &w) {
        cta = part_of(i, blk_q, blk_r);
        const uint32_t l = part_lo(cta, blk_q, blk_r), len = blk_q + (cta < blk_r ? 1u : 0u);
        if (len >= QMV_WARPS) w = part_of(i - l, len / QMV_WARPS, len % QMV_WARPS);
        else w = i - l;
    };

    const uint32_t *wbase = p.w + wb * p.w_batch_stride + t * LW;
    const uint16_t *sc = (const uint16_t *)p.scales + wb * p.s_batch_stride;
    const uint16_t *bi = (const uint16_t *)p.biases + wb * p.s_batch_stride;
    __nv_bfloat16 *out = (__nv_bfloat16 *)p.y + b * p.M * p.N;
    // nvfp4 global scale: one value, or one per expert (quantized.rs:481-490, 700-712)
    const float gmul = U::FP && p.global ? (p.expert_global ? p.global[wb] : p.global[0]) / (448.0f * 6.0f) : 1.0f;

    // Copies the scales and biases of k-chunk `chunk` of `tile` into buffer `buf` (whole warp).
    auto stage_scales = [&](int tile, int chunk, int buf) {
        const int sg0 = chunk * chunk_groups;
        if (U::FP) {
            // one scale byte per group, no biases: the two buffers share the whole per-warp area,
            // 16 rows of QMV_FPITCH bytes each
            const uint8_t *sc8 = (const uint8_t *)p.scales + wb * p.s_batch_stride;
            uint8_t *fd = reinterpret_cast<uint8_t *>(sraw) + buf * (16 * QMV_FPITCH);
            if (p.s_vec == 4) {
                const int quads = chunk_groups >> 2;
                for (int i = lane; i < 16 * quads; i += 32) {
                    const int rr = i / quads, c = i - rr * quads;
                    const int64_t at = (int64_t)min(tile * 16 + rr, last_row) * row_groups + sg0 + 4 * c;
                    cp_async<4>((uint32_t)__cvta_generic_to_shared(fd + rr * QMV_FPITCH + 4 * c), sc8 + at);
                }
            } else {
                for (int i = lane; i < 16 * chunk_groups; i += 32) {
                    const int rr = i / chunk_groups, c = i - rr * chunk_groups;
                    fd[rr * QMV_FPITCH + c] = sc8[(int64_t)min(tile * 16 + rr, last_row) * row_groups + sg0 + c];
                }
            }
            return;
        }
        uint16_t *sd = sraw + buf * 16 * QMV_SPITCH, *bd = braw + buf * 16 * QMV_SPITCH;
        if (p.s_vec == 16) {  // 16-byte copies of 8 groups
            const int chunks = chunk_groups >> 3;
            for (int i = lane; i < 16 * chunks; i += 32) {
                const int rr = i / chunks, c = i - rr * chunks;
                const int64_t at = (int64_t)min(tile * 16 + rr, last_row) * row_groups + sg0 + 8 * c;
                cp_async<16>((uint32_t)__cvta_generic_to_shared(sd + rr * QMV_SPITCH + 8 * c), sc + at);
                cp_async<16>((uint32_t)__cvta_generic_to_shared(bd + rr * QMV_SPITCH + 8 * c), bi + at);
            }
        } else if (p.s_vec == 4) {  // 4-byte copies of 2 groups
            const int pairs = chunk_groups >> 1;
            for (int i = lane; i < 16 * pairs; i += 32) {
                const int rr = i / pairs, c = i - rr * pairs;
                const int64_t at = (int64_t)min(tile * 16 + rr, last_row) * row_groups + sg0 + 2 * c;
                cp_async<4>((uint32_t)__cvta_generic_to_shared(sd + rr * QMV_SPITCH + 2 * c), sc + at);
                cp_async<4>((uint32_t)__cvta_generic_to_shared(bd + rr * QMV_SPITCH + 2 * c), bi + at);
            }
        } else {
            for (int i = lane; i < 16 * chunk_groups; i += 32) {
                const int rr = i / chunk_groups, c = i - rr * chunk_groups;
                const int64_t at = (int64_t)min(tile * 16 + rr, last_row) * row_groups + sg0 + c;
                sd[rr * QMV_SPITCH + c] = sc[at];
                bd[rr * QMV_SPITCH + c] = bi[at];
            }
        }
    };

    // Prefetch cursor: the iteration whose words are copied next.
    uint32_t pf = lo;
    int pf_tile = (int)(lo / (uint32_t)ipt), pf_it = (int)(lo - (uint32_t)pf_tile * (uint32_t)ipt);
    const int pf_tile0 = pf_tile, pf_it0 = pf_it;  // where this run starts
    const uint32_t *pf_a = nullptr, *pf_q = nullptr;
    auto pf_rows = [&]() {
        pf_a = wbase + (size_t)min(pf_tile * 16 + r, last_row) * row_words + pf_it * (4 * LW);
        pf_q = wbase + (size_t)min(pf_tile * 16 + r + 8, last_row) * row_words + pf_it * (4 * LW);
    };
    // Issues the copies of one iteration into `stage` and always commits one group, so the
    // group count seen by wait_group is the same for every lane and iteration.
    auto prefetch = [&](int stage) {
        if (pf < hi) {
#pragma unroll
            for (int c = 0; c < CPL; c++) {
                cp_async<CW * 4>(ring_s + stage * STAGE_BYTES + c * (32 * CW * 4), pf_a + c * CW);
                cp_async<CW * 4>(ring_s + stage * STAGE_BYTES + HALF_BYTES + c * (32 * CW * 4), pf_q + c * CW);
            }
            pf_a += 4 * LW;
            pf_q += 4 * LW;
            pf++;
            if (++pf_it == ipt) {
                pf_it = 0;
                pf_tile++;
                pf_rows();
            }
        }
        cp_async_commit();
    };

    // Programmatic dependent launch: the next kernel of the stream may be scheduled from now on,
    // and this one starts copying weights (which no product writes) while the kernel before it is
    // still finishing; only then does it wait for that kernel's results.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (lo < hi) {
        stage_scales(pf_tile, pf_it / ci, 0);
        pf_rows();
    }
#pragma unroll
    for (int st = 0; st < QMV_STAGES; st++) prefetch(st);
    asm volatile("griddepcontrol.wait;" ::: "memory");  // activations, scratch and output belong to this kernel from here
    // ── stage the activations once per block (the first weight copies are already in flight) ──
    {
        const uint16_t *x = (const uint16_t *)p.x + xb * p.x_batch_stride;
        const int blocks_per_row = (int)(p.K / CODES);
        const int total_blocks = p.M * blocks_per_row;
        for (int i = tid; i < total_blocks; i += QMV_THREADS) {
            const int m = i / blocks_per_row, blk = i - m * blocks_per_row;
            uint16_t in[CODES], outv[XW * 2];
            const uint16_t *src = x + (int64_t)m * p.ldx + (int64_t)blk * CODES;
            if (p.x_vec) {
                if (CODES == 4) {
                    *reinterpret_cast<uint2 *>(in) = __ldcg(reinterpret_cast<const uint2 *>(src));
                } else {
#pragma unroll
                    for (int v = 0; v < CODES / 8; v++)
                        *reinterpret_cast<uint4 *>(in + 8 * v) = __ldcg(reinterpret_cast<const uint4 *>(src) + v);
                }
            } else {
#pragma unroll
                for (int j = 0; j < CODES; j++) in[j] = src[j];
            }
            U::permute(in, outv);
            // word `blk` of the row belongs to iteration blk / (4 WPL), lane t = (blk / WPL) % 4, word j = blk % WPL
            const int it = blk / (4 * WPL), tt = (blk / WPL) & 3, j = blk % WPL;
            uint32_t *dst = xs + (size_t)m * xs_pitch + (size_t)(((it * WPL + j) * 4 + tt) * XW);
#pragma unroll
            for (int v = 0; v < XW; v++) dst[v] = (uint32_t)outv[2 * v] | ((uint32_t)outv[2 * v + 1] << 16);
        }
        if (tid < 64) zero[tid] = 0u;
        if (tid < QMV_WARPS) lcount[tid] = 0u;
    }
    __syncthreads();  // activations staged

    const bool xrow = r < p.M;
    const int x_it_step = xrow ? 4 * WPL * XW : 0;  // words per iteration in xs (0: stay on the zero page)
    const uint32_t *xbase = xrow ? xs + (size_t)r * xs_pitch + t * XW : zero + t * XW;
    int seg_count = 0;   // segments started so far (buffer parity)
    int prev_iters = 0;  // iterations of the previous segment
    int stage = 0;       // ring stage of the next iteration
    float acc[4] = {0.f, 0.f, 0.f, 0.f};  // rows r / r+8 x activation rows 2t / 2t+1
    float acd[4] = {0.f, 0.f, 0.f, 0.f};  // second accumulator: halves the MMA dependency chain

    int tile = pf_tile0, it0 = pf_it0;  // position of f in the sequence, kept without divisions
    for (uint32_t f = lo; f < hi;) {
        // Segment: the part of one k-chunk of one tile that lies in [f, hi).
        const int chunk = it0 / ci;
        const int it1 = (int)min((uint32_t)((chunk + 1) * ci), hi - f + (uint32_t)it0);
        const uint32_t f1 = f + (uint32_t)(it1 - it0);
        const int seg_buf = seg_count & 1;
        const uint16_t *sd = sraw + seg_buf * 16 * QMV_SPITCH, *bd = braw + seg_buf * 16 * QMV_SPITCH;
        // wait_group in the loop below covers a copy once QMV_STAGES groups were committed after it;
        // a shorter previous segment (or the very first one) needs an explicit wait.  Then the
        // copies of all lanes are made visible across the warp, and the next segment's scales
        // start their way into the buffer the previous segment has finished with.
        if (prev_iters <= QMV_STAGES) cp_async_wait<0>();
        __syncwarp();
        if (f1 < hi) {
            const bool wrap = it1 == ipt;
            stage_scales(wrap ? tile + 1 : tile, wrap ? 0 : it1 / ci, (seg_count + 1) & 1);
        }
        prev_iters = it1 - it0;
        seg_count++;
        const int gofs = (it0 - chunk * ci) * IK + t * (WPL * CODES);  // k offset inside the chunk
        const uint16_t *sa = sd + r * QMV_SPITCH, *sq = sd + (r + 8) * QMV_SPITCH;
        const uint16_t *ba = bd + r * QMV_SPITCH, *bq = bd + (r + 8) * QMV_SPITCH;
        const uint32_t *xp = xbase + (size_t)it0 * x_it_step;
        for (int it = it0; it < it1; it++) {
            cp_async_wait<QMV_STAGES - 1>();  // the oldest group, this iteration's words, has landed
            uint32_t wa_[LW], wq_[LW];
            {
                const uint32_t *slot = ring + (size_t)stage * (2 * 32 * LW) + lane * CW;
                if (UW == 3) {
#pragma unroll
                    for (int c = 0; c < LW; c++) {
                        wa_[c] = slot[c * 32];
                        wq_[c] = slot[32 * LW + c * 32];
                    }
                } else if (WPL == 8) {
#pragma unroll
                    for (int c = 0; c < 2; c++) {
                        uint4 a = *reinterpret_cast<const uint4 *>(slot + c * 128);
                        uint4 q = *reinterpret_cast<const uint4 *>(slot + 32 * WPL + c * 128);
                        wa_[(4 * c) % WPL] = a.x; wa_[(4 * c + 1) % WPL] = a.y; wa_[(4 * c + 2) % WPL] = a.z; wa_[(4 * c + 3) % WPL] = a.w;
                        wq_[(4 * c) % WPL] = q.x; wq_[(4 * c + 1) % WPL] = q.y; wq_[(4 * c + 2) % WPL] = q.z; wq_[(4 * c + 3) % WPL] = q.w;
                    }
                } else if (WPL == 4) {
                    uint4 a = *reinterpret_cast<const uint4 *>(slot), q = *reinterpret_cast<const uint4 *>(slot + 32 * WPL);
                    wa_[0] = a.x; wa_[1 % WPL] = a.y; wa_[2 % WPL] = a.z; wa_[3 % WPL] = a.w;
                    wq_[0] = q.x; wq_[1 % WPL] = q.y; wq_[2 % WPL] = q.z; wq_[3 % WPL] = q.w;
                } else if (WPL == 2) {
                    uint2 a = *reinterpret_cast<const uint2 *>(slot), q = *reinterpret_cast<const uint2 *>(slot + 32 * WPL);
                    wa_[0] = a.x; wa_[1 % WPL] = a.y;
                    wq_[0] = q.x; wq_[1 % WPL] = q.y;
                } else {
                    wa_[0] = slot[0];
                    wq_[0] = slot[32 * WPL];
                }
            }
            const int g = (gofs + (it - it0) * IK) >> p.gs_shift;
            GroupConsts ga, gq, ga1, gq1;  // (ga1, gq1: the second group of a lane's words, nvfp4 only)
            if (U::FP) {
                const uint8_t *fa = reinterpret_cast<const uint8_t *>(sraw) + seg_buf * (16 * QMV_FPITCH) + r * QMV_FPITCH;
                const uint8_t *fq = fa + 8 * QMV_FPITCH;
                ga.s2 = fp4_scale2(fa[g], U::FP == 1); gq.s2 = fp4_scale2(fq[g], U::FP == 1);
                ga.b2 = gq.b2 = ga.ns2 = gq.ns2 = 0u;
                ga1 = ga; gq1 = gq;
                if (U::FP == 3 && WPL * CODES > 16) {
                    ga1.s2 = fp4_scale2(fa[g + 1], false);
                    gq1.s2 = fp4_scale2(fq[g + 1], false);
                }
            } else {
                ga.s2 = (uint32_t)sa[g] * 0x10001u; ga.b2 = (uint32_t)ba[g] * 0x10001u;
                gq.s2 = (uint32_t)sq[g] * 0x10001u; gq.b2 = (uint32_t)bq[g] * 0x10001u;
                ga.ns2 = bf2_mul(ga.s2, 0xC300C300u);  // -128 s, exact
                gq.ns2 = bf2_mul(gq.s2, 0xC300C300u);
                ga1 = ga; gq1 = gq;
            }
#pragma unroll
            for (int j = 0; j < WPL; j++) {
                uint32_t ra[AREGS], rq[AREGS], xr[XW];
                const bool second = U::FP == 3 && j * CODES >= 16;  // nvfp4: 16 values per scale
                U::run(&wa_[j * UW], second ? ga1 : ga, ra);
                U::run(&wq_[j * UW], second ? gq1 : gq, rq);
                if (XW == 2) {
                    uint2 q = *reinterpret_cast<const uint2 *>(xp + j * 4 * XW);
                    xr[0] = q.x; xr[1] = q.y;
                } else {
#pragma unroll
                    for (int v = 0; v < XW; v += 4) {
                        uint4 q = *reinterpret_cast<const uint4 *>(xp + j * 4 * XW + v);
                        xr[v] = q.x; xr[v + 1] = q.y; xr[v + 2] = q.z; xr[v + 3] = q.w;
                    }
                }
#pragma unroll
                for (int h = 0; h < AREGS / 2; h++) {
                    if ((j * (AREGS / 2) + h) & 1)
                        mma_bf16_16816(acd, ra[2 * h], rq[2 * h], ra[2 * h + 1], rq[2 * h + 1], xr[2 * h], xr[2 * h + 1]);
                    else
                        mma_bf16_16816(acc, ra[2 * h], rq[2 * h], ra[2 * h + 1], rq[2 * h + 1], xr[2 * h], xr[2 * h + 1]);
                }
            }
            xp += x_it_step;
            // Refill the slot just consumed (its words are in registers and already used).
            prefetch(stage);
            stage = stage + 1 == QMV_STAGES ? 0 : stage + 1;
        }
        f = f1;
        if (it1 != ipt && f1 != hi) {  // the tile goes on in the next k-chunk
            it0 = it1;
            continue;
        }
        const int done_tile = tile;
        if (it1 == ipt) {
            tile++;
            it0 = 0;
        } else it0 = it1;

        // ── the run leaves this tile: rows r, r + 8; activation rows 2t, 2t + 1 ─────────
        float v[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            v[i] = acc[i] + acd[i];
            acc[i] = acd[i] = 0.f;
        }
        const int n0 = done_tile * 16;
        const uint32_t t_lo = (uint32_t)done_tile * (uint32_t)ipt, t_hi = t_lo + (uint32_t)ipt;
        bool store = lo <= t_lo && hi >= t_hi;  // the whole tile was this warp's
        uint32_t c1 = 0, w1 = 0, c2 = 0, w2 = 0;
        if (!store) {
            owner(t_lo, c1, w1);
            owner(t_hi - 1, c2, w2);
        }
        if (!store && c1 == c2) {
            // Every warp that holds a part of this tile belongs to this block: the partials meet in
            // shared memory.  A warp leaves at most two (the tile its run starts in and the one it
            // ends in); the warp that arrives last adds them in run order.
            float *mine = lpart + (warp * 2 + (done_tile == pf_tile0 ? 0 : 1)) * 128;
            *reinterpret_cast<float2 *>(mine + r * 8 + 2 * t) = make_float2(v[0], v[1]);
            *reinterpret_cast<float2 *>(mine + (r + 8) * 8 + 2 * t) = make_float2(v[2], v[3]);
            __threadfence_block();
            __syncwarp();
            uint32_t arrived = 0;
            if (lane == 0) arrived = atomicAdd(lcount + w1, 1u);
            arrived = __shfl_sync(0xFFFFFFFFu, arrived, 0);
            if (arrived == w2 - w1) {
                __threadfence_block();
                v[0] = v[1] = v[2] = v[3] = 0.f;
                for (uint32_t w = w1; w <= w2; w++) {
                    // warp w left this tile's partial in its slot 0 if its run starts in the tile
                    const uint32_t w_lo = blk_lo + part_lo(w, wq, wr);
                    const float *src = lpart + (w * 2 + (w_lo >= t_lo ? 0 : 1)) * 128;
                    float2 a = *reinterpret_cast<const float2 *>(src + r * 8 + 2 * t);
                    float2 q = *reinterpret_cast<const float2 *>(src + (r + 8) * 8 + 2 * t);
                    v[0] += a.x; v[1] += a.y; v[2] += q.x; v[3] += q.y;
                }
                store = true;
            }
        } else if (!store) {
            // The tile is cut by a block boundary: the warps first .. last (numbered through the
            // grid, every block of a multi-block grid runs all its warps), this one number `mine`,
            // leave their 16 x 8 partials in scratch; the one that arrives last adds them in run
            // order (so the result does not depend on arrival order) and rearms the counter.
            const int first = (int)(c1 * QMV_WARPS + w1), last = (int)(c2 * QMV_WARPS + w2);
            const int mine = (int)blockIdx.x * QMV_WARPS + warp - first, count = last - first + 1;
            const int64_t slot = b * tiles + done_tile;
            float *part = p.partials + slot * p.max_parts * 128;
            __stcg(reinterpret_cast<float2 *>(part + mine * 128 + r * 8 + 2 * t), make_float2(v[0], v[1]));
            __stcg(reinterpret_cast<float2 *>(part + mine * 128 + (r + 8) * 8 + 2 * t), make_float2(v[2], v[3]));
            __threadfence();
            __syncwarp();
            uint32_t arrived = 0;
            if (lane == 0) arrived = atomicAdd(p.counters + slot, 1u);
            arrived = __shfl_sync(0xFFFFFFFFu, arrived, 0);
            if (arrived == (uint32_t)count - 1) {
                __threadfence();
                v[0] = v[1] = v[2] = v[3] = 0.f;
                for (int s2 = 0; s2 < count; s2++) {
                    float2 a = __ldcg(reinterpret_cast<const float2 *>(part + s2 * 128 + r * 8 + 2 * t));
                    float2 q = __ldcg(reinterpret_cast<const float2 *>(part + s2 * 128 + (r + 8) * 8 + 2 * t));
                    v[0] += a.x; v[1] += a.y; v[2] += q.x; v[3] += q.y;
                }
                if (lane == 0) p.counters[slot] = 0u;
                store = true;
            }
        }
        if (store && U::FP) {
#pragma unroll
            for (int i = 0; i < 4; i++) v[i] *= gmul;
        }
        if (store && !p.peer) {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int row = n0 + r + (i >> 1) * 8, col = 2 * t + (i & 1);
                if (col < p.M && row <= last_row) out[(int64_t)col * p.N + row] = __float2bfloat16_rn(v[i]);
            }
        } else if (store) {
            // fused gather: into slot `rank` of this rank's own gathered buffer; the block that
            // finishes last sends the whole slice to the other ranks (end of the kernel)
            __nv_bfloat16 *dst = reinterpret_cast<__nv_bfloat16 *>(static_cast<char *>(p.peer->base[p.peer->rank]) + p.peer_out_offset) +
                                 (int64_t)p.peer->rank * p.M * p.N;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int row = n0 + r + (i >> 1) * 8, col = 2 * t + (i & 1);
                if (col < p.M && row <= last_row) dst[(int64_t)col * p.N + row] = __float2bfloat16_rn(v[i]);
            }
        }
    }
    cp_async_wait<0>();
    if (p.peer) {
        // The block that finishes last copies this rank's slice from its own gathered buffer into
        // every other rank's (16-byte peer stores over NVLink by all its threads), makes them
        // visible system-wide, raises this rank's flag in every region, and then waits until every
        // rank's flag in its own region shows the same product finished: when this kernel ends, the
        // gathered buffer is complete on this rank, and the next kernel of the stream needs no
        // wait of its own.  Rank r has finished n fused products when flag r holds n; this rank's
        // own count is at byte 64.  (Fences by thread 0 after a block barrier cover the whole
        // block's stores: the barrier orders them before the fence, and a fence is cumulative.)
        // The wait is bounded; when it gives up the error word says so.
        __syncthreads();
        uint32_t *own = static_cast<uint32_t *>(p.peer->base[p.peer->rank]);
        if (tid == 0) {
            __threadfence();
            lcount[QMV_WARPS] = atomicAdd(own + 17, 1u) == gridDim.x * gridDim.z - 1 ? 1u : 0u;
            __threadfence();
        }
        __syncthreads();
        if (lcount[QMV_WARPS]) {
            const size_t slice = (size_t)p.M * p.N * 2, at = p.peer_out_offset + (size_t)p.peer->rank * slice;
            const char *src = static_cast<const char *>(p.peer->base[p.peer->rank]) + at;
            // each piece is read once and stored to every peer (the reads are L2 round trips)
            if (slice % 16 == 0 && at % 16 == 0) {
                for (size_t i = (size_t)tid * 16; i < slice; i += (size_t)QMV_THREADS * 16) {
                    const uint4 piece = __ldcg(reinterpret_cast<const uint4 *>(src + i));
                    for (int rk = 0; rk < p.peer->size; rk++)
                        if (rk != p.peer->rank) *reinterpret_cast<uint4 *>(static_cast<char *>(p.peer->base[rk]) + at + i) = piece;
                }
            } else {
                for (size_t i = (size_t)tid * 2; i < slice; i += (size_t)QMV_THREADS * 2) {
                    const uint16_t piece = __ldcg(reinterpret_cast<const uint16_t *>(src + i));
                    for (int rk = 0; rk < p.peer->size; rk++)
                        if (rk != p.peer->rank) *reinterpret_cast<uint16_t *>(static_cast<char *>(p.peer->base[rk]) + at + i) = piece;
                }
            }
            __syncthreads();
            if (tid == 0) {
                const uint32_t seq = __ldcg(own + 16) + 1u;
                own[17] = 0u;
                // one release fence for all flags (a releasing store per flag would fence each time)
                asm volatile("fence.acq_rel.sys;" ::: "memory");
                for (int rk = 0; rk < p.peer->size; rk++) {
                    uint32_t *flag = static_cast<uint32_t *>(p.peer->base[rk]) + p.peer->rank;
                    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(seq) : "memory");
                }
                __stcg(own + 16, seq);
                // all flags are polled together (relaxed loads that overlap), one fence acquires
                bool all = false;
                for (uint32_t spins = 0; spins < (1u << 20) && !all; spins++) {  // about a second
                    all = true;
                    for (int rk = 0; rk < p.peer->size; rk++) {
                        uint32_t seen;
                        asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(own + rk) : "memory");
                        all = all && seen >= seq;
                    }
                }
                asm volatile("fence.acq_rel.sys;" ::: "memory");
                if (!all && p.error) *p.error = 2;
            }
        }
    }
}

// ── host side ──────────────────────────────────────────────────────────────────────────

// A unit is the smallest run of words that holds whole codes: one word, or three for 3 and 6 bits.
// (`bits` below is the kernel's kind: the affine bit width, or 40 = mxfp4, 41 = nvfp4.)
static bool kind_fp(int bits) { return bits == 40 || bits == 41; }
static int code_bits(int bits) { return kind_fp(bits) ? 4 : bits; }
static int unit_words(int bits) { return bits == 3 || bits == 6 ? 3 : 1; }
static int codes_per_word(int bits) { return unit_words(bits) * 32 / code_bits(bits); }  // codes per unit
int qmv_kind(int32_t mode, int32_t bits) {
    if (mode == NVC_AFFINE) return bits;
    if (mode == NVC_MXFP4 && bits == 4) return 40;
    if (mode == NVC_NVFP4 && bits == 4) return 41;
    return 0;
}

// Words per lane per iteration: the widest vector load whose 4-lane span divides K.  Eight words
// (two 16-byte copies) execute fewer instructions per weight but issue slower on the B200 than
// four; they stay selectable with NUVEC_QMV_MAX_WPL=8.
static int wpl_for(int bits, int gs, int64_t K) {
    if (bits != 2 && bits != 3 && bits != 4 && bits != 6 && bits != 8 && !kind_fp(bits)) return 0;
    const int codes = codes_per_word(bits);
    static const int cap = [] { const char *e = getenv("NUVEC_QMV_MAX_WPL"); return e && *e ? atoi(e) : 4; }();
    const int span = bits == 41 ? 2 * gs : gs;   // nvfp4 lanes may hold two groups of 16
    for (int wpl = bits == 3 ? 1 : bits == 2 || bits == 6 ? 2 : kind_fp(bits) ? 4 : 8; wpl >= 1; wpl >>= 1) {
        if (wpl > cap) continue;
        if (wpl * codes > span) continue;        // a lane's words stay inside one group
        if (K % (4 * wpl * codes) == 0) return wpl;
    }
    return 0;
}

static size_t qmv_smem(int M, int64_t K, int bits, int wpl) {
    const int codes = codes_per_word(bits), xw = codes / 2, lw = wpl * unit_words(bits);
    return (size_t)(M * (K / codes * xw + 16) + 64 + QMV_WARPS * (2 * 16 * QMV_SPITCH) +
                    qmv_stages(wpl) * 2 * QMV_THREADS * lw + QMV_WARPS * 2 * 128 + QMV_WARPS + 4) * 4 + 16;
}

bool qmv_affine_eligible(int32_t mode, int32_t gs, int32_t bits, int32_t dtype, int32_t transpose, int64_t M,
                         int64_t N, int64_t K, const void *x, int64_t ldx, int64_t x_batch_stride, const uint32_t *w,
                         int64_t w_batch_stride) {
    (void)x; (void)ldx; (void)x_batch_stride;
    if (dtype != NVC_BF16 || !transpose) return false;
    bits = qmv_kind(mode, bits);
    if (bits == 0) return false;
    if (M < 1 || M > 8 || N < 1 || K < gs) return false;
    int wpl = wpl_for(bits, gs, K);
    if (wpl == 0) return false;
    int64_t row_words = K * code_bits(bits) / 32;
    const int cw = unit_words(bits) == 3 ? 1 : wpl == 8 ? 4 : wpl;  // words per asynchronous copy
    if (row_words % cw != 0 || w_batch_stride % cw != 0 || ((uintptr_t)w % (4 * cw)) != 0) return false;
    if (((N + 15) / 16) * (K / (4 * wpl * codes_per_word(bits))) >= (int64_t)1 << 30) return false;  // 32-bit iteration counts
    return qmv_smem((int)M, K, bits, wpl) <= 220 * 1024;  // all activations are staged in shared memory
}

template <int BITS, int WPL>
static int32_t launch_qmv_cfg(nvc_device *dev, QmvParams &p, dim3 grid, size_t smem) {
    auto kernel = qmv_affine_kernel<BITS, WPL>;
    static size_t configured = 0;  // largest dynamic shared memory size set so far (per instantiation)
    if (smem > 48 * 1024 && smem > configured) {
        NVC_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = smem;
    }
    // Launched with programmatic stream serialization: the kernel may start while its predecessor
    // drains and synchronises with it on the device (griddepcontrol.wait) before it reads
    // activations or writes anything.  NUVEC_PDL=0 restores plain stream order.
    static const bool pdl = [] { const char *e = getenv("NUVEC_PDL"); return !(e && *e == '0'); }();
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(QMV_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = dev->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    NVC_CUDA(cudaLaunchKernelEx(&cfg, kernel, p));
    return check_launch(dev, "qmv_affine_kernel");
}

static int64_t env_int(const char *name, int64_t fallback) {
    const char *e = getenv(name);
    return e && *e ? atoll(e) : fallback;
}

int32_t launch_qmv_affine(nvc_device *dev, int32_t bits, QmvParams p, int64_t batch, const QmvScratch *fixed) {
    if (batch == 0 || p.N == 0 || p.M == 0) return NVC_OK;
    if (batch > 65535) return set_error(NVC_ERR_UNSUPPORTED, "qmv: %lld batches exceed the grid limit", (long long)batch);
    const int wpl = wpl_for(bits, p.gs, p.K);
    const int codes = codes_per_word(bits);
    const int ik = 4 * wpl * codes;
    p.gs_shift = p.gs == 16 ? 4 : p.gs == 32 ? 5 : p.gs == 64 ? 6 : 7;
    const int64_t tiles = (p.N + 15) / 16, ipt = p.K / ik, total = tiles * ipt;
    // k-chunk for staging scales: the largest divisor of K that holds whole iterations and whole
    // groups, up to the groups the staging area takes (and 2048 values).
    const int64_t max_groups = kind_fp(bits) ? QMV_FP_SEG_GROUPS : QMV_SEG_GROUPS;
    int64_t chunk = max_groups * p.gs;
    if (chunk > 2048) chunk = 2048;
    const int64_t unit = ik > p.gs ? ik : p.gs;  // both are powers of two: the larger is their common multiple
    chunk = chunk / unit * unit;
    while (chunk > unit && p.K % chunk != 0) chunk -= unit;
    if (chunk < unit || p.K % chunk != 0) chunk = unit;
    p.chunk_k = (int32_t)chunk;
    {
        // Widest aligned copy for staging scales and biases: 8 groups, 2 groups or single loads
        // (4-bit floating point: 4 scale bytes or single loads).
        const int64_t rg = p.K / p.gs, cg = chunk / p.gs;
        const uintptr_t al = (uintptr_t)p.scales | (uintptr_t)p.biases;
        if (kind_fp(bits)) p.s_vec = (al % 4 == 0 && p.s_batch_stride % 4 == 0 && rg % 4 == 0 && cg % 4 == 0) ? 4 : 0;
        else if (al % 16 == 0 && p.s_batch_stride % 8 == 0 && rg % 8 == 0 && cg % 8 == 0) p.s_vec = 16;
        else if (al % 4 == 0 && p.s_batch_stride % 2 == 0 && rg % 2 == 0 && cg % 2 == 0) p.s_vec = 4;
        else p.s_vec = 0;
    }
    const size_t smem = qmv_smem(p.M, p.K, bits, wpl);
    // Blocks: as many as stay resident (two per multiprocessor while shared memory allows), but
    // no more than give every warp a few iterations.
    // (each block also takes 1 KB of shared memory the system reserves)
    int64_t per_sm = (int64_t)(227 * 1024) / (int64_t)(smem + 1024);
    if (per_sm > QMV_BLOCKS_PER_SM) per_sm = QMV_BLOCKS_PER_SM;
    if (per_sm < 1) per_sm = 1;
    per_sm = env_int("NUVEC_QMV_PER_SM", per_sm);
    int64_t blocks = per_sm * dev->prop.multiProcessorCount / batch;
    const int64_t min_iters = env_int("NUVEC_QMV_MIN_ITERS", 4);
    const int64_t useful = (total + QMV_WARPS * min_iters - 1) / (QMV_WARPS * min_iters);
    if (blocks > useful) blocks = useful;
    const int64_t env_blocks = env_int("NUVEC_QMV_BLOCKS", 0);
    if (env_blocks > 0) blocks = env_blocks;
    else if (env_int("NUVEC_QMV_ALIGN", 1) != 0 && blocks > 1) {
        // A tile cut by a block boundary costs its warps a round trip through scratch; one cut between
        // warps of a block is settled in shared memory.  So, while blocks hold only a few tiles,
        // prefer a block count that divides the tiles if one lies within two fifths of the
        // resident blocks (long runs amortise the round trip and want every block).
        for (int64_t b = blocks; tiles < 4 * blocks && b * 5 >= blocks * 3 && b >= 1; b--)
            if (tiles % b == 0) {
                blocks = b;
                break;
            }
    }
    // Every block of a multi-block grid runs all its warps (the kernel numbers the warps that meet
    // in a tile through the grid).
    if (blocks > total / QMV_WARPS) blocks = total / QMV_WARPS;
    if (blocks < 1) blocks = 1;
    // Tiles cut by block boundaries: at most ipt / (shortest warp run) + 2 runs meet in one tile.
    const int64_t run = total / blocks / QMV_WARPS > 0 ? total / blocks / QMV_WARPS : 1;
    p.max_parts = (int32_t)(ipt / run + 2);
    p.blk_q = (uint32_t)(total / blocks);
    p.blk_r = (uint32_t)(total % blocks);
    const size_t partial_bytes = (size_t)tiles * batch * p.max_parts * 128 * sizeof(float);
    if (fixed) {
        // Scratch of fixed capacity provided by the caller of this function: nothing is allocated.
        if (partial_bytes > fixed->partial_bytes || (size_t)(tiles * batch) > fixed->counters_len)
            return set_error(NVC_ERR_UNSUPPORTED,
                             "qmv: this product needs %zu bytes of partial sums and %lld counters; the fixed scratch holds "
                             "%zu bytes and %zu counters", partial_bytes, (long long)(tiles * batch), fixed->partial_bytes,
                             fixed->counters_len);
        p.partials = fixed->partials;
        p.counters = fixed->counters;
    } else {
        void *scratch = nullptr;
        NVC_TRY(ensure_scratch(dev, partial_bytes, &scratch));
        p.partials = (float *)scratch;
        NVC_TRY(ensure_counters(dev, (size_t)(tiles * batch), &p.counters));
    }
    dim3 grid((unsigned)blocks, 1, (unsigned)batch);
#define NVC_QMV(B, W) if (bits == B && wpl == W) return launch_qmv_cfg<B, W>(dev, p, grid, smem);
    NVC_QMV(4, 1) NVC_QMV(4, 2) NVC_QMV(4, 4) NVC_QMV(4, 8) NVC_QMV(8, 1) NVC_QMV(8, 2) NVC_QMV(8, 4) NVC_QMV(8, 8)
    NVC_QMV(2, 1) NVC_QMV(2, 2) NVC_QMV(3, 1) NVC_QMV(6, 1) NVC_QMV(6, 2)
    NVC_QMV(40, 1) NVC_QMV(40, 2) NVC_QMV(40, 4) NVC_QMV(41, 1) NVC_QMV(41, 2) NVC_QMV(41, 4)
#undef NVC_QMV
    return set_error(NVC_ERR_UNSUPPORTED, "qmv: no kernel for %d bits, group size %d", bits, p.gs);
}

}  // namespace nvc

// ── the entry point that allocates nothing ─────────────────────────────────────────────────
//
// Scratch for nvc_quantized_matmul_noalloc: part of the library image, so every GPU that loads
// the library holds these 4 MiB until the process exits.  Layout: float32 partial sums, then the
// arrival counters.
namespace {
constexpr size_t NOALLOC_SCRATCH_BYTES = 4u << 20;
constexpr size_t NOALLOC_COUNTERS = 16384;  // one per 16-row tile: N up to 262144
constexpr size_t NOALLOC_PARTIAL_BYTES = NOALLOC_SCRATCH_BYTES - NOALLOC_COUNTERS * sizeof(uint32_t);
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_SCRATCH_BYTES];

constexpr int NOALLOC_MAX_DEVICES = 64;
std::mutex g_noalloc_mu;
void *g_noalloc_ptr[NOALLOC_MAX_DEVICES] = {};  // device address of the array, per device ordinal
}  // namespace

extern "C" int32_t nvc_quantized_matmul_noalloc(nvc_device *dev, const nvc_quant *q, const void *x, const uint32_t *w,
                                                const void *scales, const void *biases, int64_t M, int64_t N, int64_t K,
                                                void *y) {
    using namespace nvc;
    NVC_TRY(make_current(dev));
    NVC_TRY(check_quant("quantized_matmul", q));
    if (q->mode != NVC_AFFINE || !biases)
        return set_error(NVC_ERR_UNSUPPORTED, "quantized_matmul (no-alloc): affine weights with biases only");
    if (M < 0 || N < 0 || K < 0 || K % q->group_size != 0)
        return set_error(NVC_ERR_INVALID_ARGUMENT, "quantized_matmul (no-alloc): invalid shape [%lld, %lld] x [%lld, %lld]",
                         (long long)M, (long long)K, (long long)N, (long long)K);
    if (M == 0 || N == 0) return NVC_OK;
    if (!x || !w || !scales || !y) return set_error(NVC_ERR_INVALID_ARGUMENT, "quantized_matmul (no-alloc): null operand");
    if (!qmv_affine_eligible(q->mode, q->group_size, q->bits, NVC_BF16, 1, M, N, K, x, K, 0, w, 0))
        return set_error(NVC_ERR_UNSUPPORTED,
                         "quantized_matmul (no-alloc): takes bfloat16 x with 1 to 8 rows and 2-, 3-, 4-, 6- or 8-bit weights whose "
                         "rows are a whole number of 32-value iterations (got M = %lld, K = %lld, %d bits)",
                         (long long)M, (long long)K, q->bits);
    if (dev->ordinal < 0 || dev->ordinal >= NOALLOC_MAX_DEVICES)
        return set_error(NVC_ERR_UNSUPPORTED, "quantized_matmul (no-alloc): device ordinal %d", dev->ordinal);
    void *base = nullptr;
    {
        // Set-up, once per device and with that device current: the array's name is only a host-side
        // handle for the symbol, the kernel needs its address on this device.
        std::lock_guard<std::mutex> g(g_noalloc_mu);
        if (!g_noalloc_ptr[dev->ordinal]) {
            void *ptr = nullptr;
            NVC_CUDA(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
            g_noalloc_ptr[dev->ordinal] = ptr;
        }
        base = g_noalloc_ptr[dev->ordinal];
    }
    QmvScratch fixed;
    fixed.partials = reinterpret_cast<float *>(base);
    fixed.partial_bytes = NOALLOC_PARTIAL_BYTES;
    fixed.counters = reinterpret_cast<uint32_t *>(static_cast<unsigned char *>(base) + NOALLOC_PARTIAL_BYTES);
    fixed.counters_len = NOALLOC_COUNTERS;
    const int64_t tiles = (N + 15) / 16;
    if ((size_t)tiles > NOALLOC_COUNTERS)
        return set_error(NVC_ERR_UNSUPPORTED, "quantized_matmul (no-alloc): N = %lld exceeds the fixed scratch (at most %zu rows)",
                         (long long)N, NOALLOC_COUNTERS * 16);
    // The array keeps whatever the last call left; the counters must start at zero.
    NVC_CUDA(cudaMemsetAsync(fixed.counters, 0, (size_t)tiles * sizeof(uint32_t), dev->stream));
    QmvParams p{};
    p.x = x; p.w = w; p.scales = scales; p.biases = biases; p.lhs = nullptr; p.rhs = nullptr; p.y = y;
    p.N = N; p.K = K; p.ldx = K;
    p.x_batch_stride = 0; p.w_batch_stride = 0; p.s_batch_stride = 0;
    p.M = (int32_t)M; p.gs = q->group_size;
    p.x_vec = ((uintptr_t)x % 16 == 0) && (K % 8 == 0);
    return launch_qmv_affine(dev, q->bits, p, 1, &fixed);
}
