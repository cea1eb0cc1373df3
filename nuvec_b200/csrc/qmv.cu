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

#include <utility>

namespace nvc {

// ── optional timeline of the few-row kernel (diagnostic builds only: -DNUVEC_TIMELINE) ─────────
// Every launch of qmv_affine_kernel records %globaltimer at six points -- block start, before and
// after the dependency wait, activations staged, a warp's last iteration done, block end -- as the
// minimum and maximum over its blocks (warps for the fifth).  The last block to finish moves on to
// the next record.  nvc_debug_timeline_reset / _read (end of this file) clear and fetch the records.
#ifdef NUVEC_TIMELINE
constexpr int TIMELINE_RECORDS = 4096, TIMELINE_POINTS = 6;
__device__ unsigned long long g_timeline[TIMELINE_RECORDS][2 * TIMELINE_POINTS];
__device__ unsigned int g_timeline_at, g_timeline_done;
__device__ __forceinline__ unsigned long long global_timer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void timeline_put(unsigned int rec, int point, unsigned long long t) {
    atomicMin(&g_timeline[rec][2 * point], t);
    atomicMax(&g_timeline[rec][2 * point + 1], t);
}
#define QMV_TIMELINE_BEGIN unsigned long long tl_[4]; tl_[0] = global_timer();
#define QMV_TIMELINE_MARK(k) tl_[k] = global_timer();
#define QMV_TIMELINE_END(worked)                                                                         \
    {                                                                                                    \
        const unsigned int rec_ = *(volatile unsigned int *)&g_timeline_at % TIMELINE_RECORDS;           \
        if ((threadIdx.x & 31) == 0 && (worked)) timeline_put(rec_, 4, global_timer());                  \
        __syncthreads();                                                                                 \
        if (threadIdx.x == 0) {                                                                          \
            for (int k_ = 0; k_ < 4; k_++) timeline_put(rec_, k_, tl_[k_]);                              \
            timeline_put(rec_, 5, global_timer());                                                       \
            __threadfence();                                                                             \
            if (atomicAdd(&g_timeline_done, 1u) == gridDim.x * gridDim.y * gridDim.z - 1) {              \
                g_timeline_done = 0;                                                                     \
                __threadfence();                                                                         \
                g_timeline_at = g_timeline_at + 1;                                                       \
            }                                                                                            \
        }                                                                                                \
    }
#else
#define QMV_TIMELINE_BEGIN
#define QMV_TIMELINE_MARK(k)
#define QMV_TIMELINE_END(worked)
#endif

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
    if (p.rhs) {  // indices past the end select the last batch (the reference's `take` clamps, kernels.rs:120-129)
        wb = min(p.rhs[b], p.experts - 1u);
        xb = p.lhs ? (int64_t)min(p.lhs[b], p.x_batches - 1u) : b;
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
    if (p.rhs) {  // indices past the end select the last batch (the reference's `take` clamps, kernels.rs:120-129)
        wb = min(p.rhs[b], p.experts - 1u);
        xb = p.lhs ? (int64_t)min(p.lhs[b], p.x_batches - 1u) : b;
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
// 8-bit floating point (kernel "bits" 42 = mxfp8: E4M3 codes, one E8M0 scale per 32 values).  The code's
// seven magnitude bits become exponent[3:0] and mantissa[6:4] of a bfloat16 whose value is the
// magnitude * 2^-120 (the subnormal codes included: they are bfloat16 subnormals); multiplying by 2^120
// restores the value (4 significant bits) and the scale is a power of two: the operand equals the
// reference's float32 decode (crates/nuvec-core/src/kernels.rs:976-1009, fp8.rs:39-44).  The two NaN
// codes (0x7F, 0xFF), which the reference's quantizer never writes (it saturates at 448), read as 480.
// register 0 = codes (0, 2), register 1 = codes (1, 3), as for 8-bit affine.
template <> struct Unpack<42> {
    static constexpr int WBITS = 8, FP = 1;
    static constexpr int UW = 1;
    static constexpr int CODES = 4;
    static constexpr int AREGS = 2;
    static __device__ __forceinline__ void run(const uint32_t *u, const GroupConsts &c, uint32_t (&r)[2]) {
        const uint32_t w = u[0];
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const uint32_t x = w >> (8 * i);  // bytes i and i + 2 in the low byte of each half
            const uint32_t bits = lop3_and_or(x << 8, 0x80008000u, (x << 4) & 0x07F007F0u);
            r[i] = bf2_mul(bf2_mul(bits, 0x7B807B80u), c.s2);
        }
    }
    static __device__ __forceinline__ void permute(const uint16_t *x, uint16_t *out) { Unpack<8>::permute(x, out); }
};
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
// Words of the all-zero page that lanes of activation rows >= M read instead of activations: four
// iterations' worth, so that such a lane needs no address update inside a round of four.
__host__ __device__ constexpr int qmv_zero_words(int wpl, int xw) { return 16 * wpl * xw < 64 ? 64 : 16 * wpl * xw; }
// Most groups whose scale/bias are staged at a time (one k-chunk of a tile).
constexpr int QMV_SEG_GROUPS = 16;
// Row pitch (bfloat16 elements) of the staged scales: 48 bytes = 12 banks, a multiple of 16 bytes
// (the widest copy); the 8 rows a warp reads together fall on different banks.
constexpr int QMV_SPITCH = QMV_SEG_GROUPS + 8;
// 4-bit floating point: up to 64 groups (bytes) of a row per k-chunk, rows 80 bytes apart (20 banks:
// the 8 rows a warp reads together fall on different banks); 2 x 16 x 80 bytes fit the same area.
constexpr int QMV_FP_SEG_GROUPS = 64;
constexpr int QMV_FPITCH = 80;
// Per-warp scale area (bytes).  Affine: the raw scales and biases of the next k-chunk as they are
// copied from global memory (2 x 16 rows x QMV_SPITCH bf16), then the current chunk's constants
// repacked per (group, row) as the pairs {s, s}, {b, b} the dequantization consumes: QMV_SEG_GROUPS
// groups, QMV_PKPITCH bytes apart (16 rows x 8 bytes + 32: two neighbouring groups read together by a
// half-warp fall on different banks).  4-bit floating point: two buffers of 16 x QMV_FPITCH bytes.
constexpr int QMV_PKPITCH = 16 * 8 + 32;
constexpr int QMV_RAW_BYTES = 2 * 16 * QMV_SPITCH * 2;
constexpr int QMV_SCALE_AREA = 4096;
static_assert(QMV_RAW_BYTES + QMV_SEG_GROUPS * QMV_PKPITCH <= QMV_SCALE_AREA, "raw and repacked scales fit the per-warp scale area");
static_assert(2 * 16 * QMV_FPITCH <= QMV_SCALE_AREA, "the floating-point scale buffers fit the per-warp scale area");

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
//   scale area (QMV_SCALE_AREA bytes)     raw scales / biases of the next k-chunk and the repacked
//                                         constants of the current one (see QMV_PKPITCH)
//   ring  [stages][2][32] x WPL u32       packed words in flight: slot (stage, row half, lane);
//                                         WPL = 8 keeps its two 16-byte chunks 512 bytes apart
//                                         (chunk, lane) so that a quarter-warp reads 128
//                                         consecutive bytes
//   lpart [QMV_WARPS][2][128] f32         partial sums of tiles cut between warps of this block
//   lcount[QMV_WARPS + 4 + 32] u32        their arrival counters; fused collectives: word QMV_WARPS + 1 the product's
//                                         sequence number, words QMV_WARPS + 4 .. the ranks' region addresses
// Shared-memory loads by 32-bit shared address plus a compile-time offset (the main loop keeps a
// few base addresses in registers and reaches everything else through the offset field).
template <int OFS> __device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4 + %5];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a), "n"(OFS));
    return v;
}
template <int OFS> __device__ __forceinline__ uint2 lds64(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2 + %3];\n" : "=r"(v.x), "=r"(v.y) : "r"(a), "n"(OFS));
    return v;
}
template <int OFS> __device__ __forceinline__ uint32_t lds32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1 + %2];\n" : "=r"(v) : "r"(a), "n"(OFS));
    return v;
}
template <int OFS> __device__ __forceinline__ uint32_t lds_u8(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u8 %0, [%1 + %2];\n" : "=r"(v) : "r"(a), "n"(OFS));
    return v;
}
template <int OFS> __device__ __forceinline__ void sts64(uint32_t a, uint32_t x, uint32_t y) {
    asm volatile("st.shared.v2.u32 [%0 + %1], {%2, %3};\n" ::"r"(a), "n"(OFS), "r"(x), "r"(y) : "memory");
}
// cp_async with compile-time offsets on both addresses.
template <int BYTES, int SOFS, int GOFS> __device__ __forceinline__ void cp_async_at(uint32_t smem_addr, const void *gptr) {
    if (BYTES == 16)
        asm volatile("cp.async.cg.shared.global [%0 + %2], [%1 + %3], 16;\n" ::"r"(smem_addr), "l"(gptr), "n"(SOFS), "n"(GOFS) : "memory");
    else if (BYTES == 8)
        asm volatile("cp.async.ca.shared.global [%0 + %2], [%1 + %3], 8;\n" ::"r"(smem_addr), "l"(gptr), "n"(SOFS), "n"(GOFS) : "memory");
    else
        asm volatile("cp.async.ca.shared.global [%0 + %2], [%1 + %3], 4;\n" ::"r"(smem_addr), "l"(gptr), "n"(SOFS), "n"(GOFS) : "memory");
}
// f(integral_constant<int, 0>) ... f(integral_constant<int, N - 1>): a loop whose index is a constant
// expression inside the body (offsets of the loads above).
template <class F, int... Is> __device__ __forceinline__ void static_for_impl(F &&f, std::integer_sequence<int, Is...>) {
    (f(std::integral_constant<int, Is>{}), ...);
}
template <int N, class F> __device__ __forceinline__ void static_for(F &&f) {
    static_for_impl(f, std::make_integer_sequence<int, N>{});
}

// Partial sums of a tile that a run boundary cuts.  Kept out of line: only such tiles come here, and
// the main loop's registers stay free of it.  `v` holds this warp's partial sums (rows r / r + 8 x
// activation rows 2t / 2t + 1); returns true, with the complete sums in `v`, in the warp that
// arrives last at the tile, which then stores the result.
struct QmvCut {
    uint32_t lo, hi;            // this warp's run
    uint32_t blk_lo, blk_len;   // this block's run
    uint32_t wq, wr;            // the block's warps hold wq iterations, the first wr one more
    uint32_t blk_q, blk_r;      // the grid's blocks hold blk_q iterations, the first blk_r one more
    uint32_t t_lo, t_hi;        // the tile's iterations
    int32_t warp, lane, first_tile;  // first_tile: 1 when the tile is the one the warp's run starts in
    int32_t max_parts;
    float *lpart;
    uint32_t *lcount;
    float *partials;            // global scratch: [batch * blocks][max_parts][128] float32
    uint32_t *counters;         // global scratch: [batch * blocks] arrival counters
    int64_t slot0;              // batch * blocks: a tile cut by block boundaries uses the slot of its first block
};
__device__ __noinline__ bool qmv_meet_partials(const QmvCut c, float4 &v) {
    const int lane = c.lane, r = lane >> 2, t = lane & 3, warp = c.warp;
    auto part_lo = [](uint32_t i, uint32_t q, uint32_t rm) { return i * q + min(i, rm); };
    auto part_of = [](uint32_t at, uint32_t q, uint32_t rm) {
        const uint32_t big = rm * (q + 1u);
        return at < big ? at / (q + 1u) : rm + (at - big) / q;
    };
    if (c.t_lo >= c.blk_lo && c.t_hi <= c.blk_lo + c.blk_len) {
        // Every warp that holds a part of this tile belongs to this block: the partials meet in
        // shared memory.  A warp leaves at most two (the tile its run starts in and the one it
        // ends in); the warp that arrives last adds them in run order.  The tile's first and last
        // warp are found by walking from this warp's run, a step per warp and no division.
        uint32_t l = c.lo, h = c.hi, w1 = (uint32_t)warp, w2 = (uint32_t)warp;
        while (l > c.t_lo) {
            w1--;
            l -= c.wq + (w1 < c.wr ? 1u : 0u);
        }
        while (h < c.t_hi) {
            w2++;
            h += c.wq + (w2 < c.wr ? 1u : 0u);
        }
        float *mine = c.lpart + (warp * 2 + (c.first_tile ? 0 : 1)) * 128;
        *reinterpret_cast<float2 *>(mine + r * 8 + 2 * t) = make_float2(v.x, v.y);
        *reinterpret_cast<float2 *>(mine + (r + 8) * 8 + 2 * t) = make_float2(v.z, v.w);
        __threadfence_block();
        __syncwarp();
        uint32_t arrived = 0;
        if (lane == 0) arrived = atomicAdd(c.lcount + w1, 1u);
        arrived = __shfl_sync(0xFFFFFFFFu, arrived, 0);
        if (arrived != w2 - w1) return false;
        __threadfence_block();
        v = make_float4(0.f, 0.f, 0.f, 0.f);
        for (uint32_t w = w1; w <= w2; w++) {
            // warp w left this tile's partial in its slot 0 if its run starts in the tile
            const uint32_t w_lo = c.blk_lo + part_lo(w, c.wq, c.wr);
            const float *src = c.lpart + (w * 2 + (w_lo >= c.t_lo ? 0 : 1)) * 128;
            float2 a = *reinterpret_cast<const float2 *>(src + r * 8 + 2 * t);
            float2 q = *reinterpret_cast<const float2 *>(src + (r + 8) * 8 + 2 * t);
            v.x += a.x; v.y += a.y; v.z += q.x; v.w += q.y;
        }
        return true;
    }
    // The tile is cut by a block boundary: the warps first .. last (numbered through the grid, every
    // block of a multi-block grid runs all its warps), this one number `mine`, leave their 16 x 8
    // partials in scratch; the one that arrives last adds them in run order (so the result does not
    // depend on arrival order) and rearms the counter.
    auto owner = [&](uint32_t i, uint32_t &cta) {  // number, through the grid, of the warp whose run holds iteration i
        cta = part_of(i, c.blk_q, c.blk_r);
        const uint32_t l = part_lo(cta, c.blk_q, c.blk_r), len = c.blk_q + (cta < c.blk_r ? 1u : 0u);
        const uint32_t w = len >= QMV_WARPS ? part_of(i - l, len / QMV_WARPS, len % QMV_WARPS) : i - l;
        return (int)(cta * QMV_WARPS + w);
    };
    uint32_t cta_first = 0, cta_last = 0;
    const int first = owner(c.t_lo, cta_first), last = owner(c.t_hi - 1, cta_last);
    const int mine = (int)blockIdx.x * QMV_WARPS + warp - first, count = last - first + 1;
    // The tile's first block is the first block of no other tile cut by a block boundary (the tile
    // before it, if cut, starts in an earlier block): its number names the tile's slot.
    const int64_t slot = c.slot0 + cta_first;
    float *part = c.partials + slot * c.max_parts * 128;
    uint32_t *counter = c.counters + slot;
    __stcg(reinterpret_cast<float2 *>(part + mine * 128 + r * 8 + 2 * t), make_float2(v.x, v.y));
    __stcg(reinterpret_cast<float2 *>(part + mine * 128 + (r + 8) * 8 + 2 * t), make_float2(v.z, v.w));
    __threadfence();
    __syncwarp();
    uint32_t arrived = 0;
    if (lane == 0) arrived = atomicAdd(counter, 1u);
    arrived = __shfl_sync(0xFFFFFFFFu, arrived, 0);
    if (arrived != (uint32_t)count - 1) return false;
    __threadfence();
    v = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s2 = 0; s2 < count; s2++) {
        float2 a = __ldcg(reinterpret_cast<const float2 *>(part + s2 * 128 + r * 8 + 2 * t));
        float2 q = __ldcg(reinterpret_cast<const float2 *>(part + s2 * 128 + (r + 8) * 8 + 2 * t));
        v.x += a.x; v.y += a.y; v.z += q.x; v.w += q.y;
    }
    if (lane == 0) *counter = 0u;
    return true;
}

template <int BITS, int WPL>
__global__ void __launch_bounds__(QMV_THREADS, QMV_BLOCKS_PER_SM) qmv_affine_kernel(QmvParams p) {
    using U = Unpack<BITS>;
    constexpr int CODES = U::CODES, AREGS = U::AREGS, UW = U::UW;
    constexpr int LW = WPL * UW;               // words per lane, row half and iteration (WPL units of UW words)
    constexpr int IK = 4 * WPL * CODES;
    constexpr int XW = AREGS;  // activation words per unit (AREGS bf16 pairs)
    constexpr int QMV_STAGES = qmv_stages(WPL);
    // 3-word units (3- and 6-bit codes): a lane's words are only 4-byte aligned, so the copies do not
    // follow the lanes.  A stage holds the tile's 16 row pieces one after the other (ROWB bytes each, a
    // multiple of 48), two lanes copy a row piece in 16-byte parts, and lane 4 r + t finds its LW words
    // at r * ROWB + t * LW * 4: the lanes' words lie back to back, LW words per lane.
    constexpr bool ROWMAJOR = UW == 3;
    constexpr int ROWB = 4 * LW * 4;           // bytes of one row piece
    // copies per lane and row half (other formats)
    constexpr int CPL = WPL == 8 ? 2 : 1;
    constexpr int CW = ROWMAJOR ? LW : LW / CPL;  // words per copy (3-word units: words per lane)
    extern __shared__ __align__(16) uint32_t smem[];
    QMV_TIMELINE_BEGIN

    const int tid = threadIdx.x, lane = tid & 31;
    // the warp index read from lane 0: the compiler then knows that everything derived from it (run
    // bounds, loop trip counts) is the same for the whole warp and keeps mma.sync free of re-convergence code
    const int warp = __shfl_sync(0xFFFFFFFFu, tid >> 5, 0);
    const int r = lane >> 2, t = lane & 3;
    const int64_t b = blockIdx.z;
    int64_t xb = b, wb = b;
    if (p.rhs) {
        // indices past the end select the last expert / activation batch, as the reference's `take`
        // clamps them (crates/nuvec-core/src/kernels.rs:120-129)
        wb = min(p.rhs[b], p.experts - 1u);
        xb = p.lhs ? (int64_t)min(p.lhs[b], p.x_batches - 1u) : b;
    }
    // Everything the loops divide by comes from the host: the kernel itself never divides on its
    // per-iteration or per-chunk paths.
    const int row_groups = p.row_groups;    // K / group size
    const uint32_t row_words = p.row_words; // K * bits / 32
    const int ipt = p.ipt;                  // iterations per tile, K / IK
    const int ci = p.ci;                    // iterations per k-chunk (scales are staged per chunk)
    const int chunk_groups = p.chunk_groups;
    const int tiles = p.tiles;
    const int last_row = (int)p.N - 1;

    const int xs_pitch = p.xs_pitch;  // words; = 16 (mod 32) keeps two rows on disjoint banks
    constexpr int X_IT_WORDS = 4 * WPL * XW;              // activation words of one iteration (one row)
    constexpr int ZERO_WORDS = qmv_zero_words(WPL, XW);   // four iterations' worth: lanes of rows >= M never leave it
    uint32_t *xs = smem;
    uint32_t *zero = xs + (size_t)p.M * xs_pitch;
    uint16_t *sraw = reinterpret_cast<uint16_t *>(zero + ZERO_WORDS) + (size_t)warp * (QMV_SCALE_AREA / 2);
    uint16_t *braw = sraw + 16 * QMV_SPITCH;
    uint32_t *ring = zero + ZERO_WORDS + QMV_WARPS * (QMV_SCALE_AREA / 4) + (size_t)warp * (QMV_STAGES * 2 * 32 * LW);
    const uint32_t ring_s = (uint32_t)__cvta_generic_to_shared(ring + lane * CW);
    // 3-word units: where this lane's copies go (row piece lane / 2, its first or second half)
    constexpr int HB = ROWB / 2 / 16 * 16;     // where the second lane of a row piece starts: 16 (3 words) or 48 (6 words)
    constexpr int PARTS = LW == 3 ? 1 : 3;     // 16-byte parts every lane copies; with 3 words the first lane of a
    const bool extra_part = LW == 3 && (lane & 1) == 0;  // row piece copies one more, 32 bytes on
    const uint32_t copy_s = (uint32_t)__cvta_generic_to_shared(ring) + (uint32_t)((lane >> 1) * ROWB + (lane & 1) * HB);
    const uint32_t sraw_s = (uint32_t)__cvta_generic_to_shared(sraw);
    float *lpart = reinterpret_cast<float *>(ring + (size_t)(QMV_WARPS - warp) * (QMV_STAGES * 2 * 32 * LW));
    uint32_t *lcount = reinterpret_cast<uint32_t *>(lpart + QMV_WARPS * 2 * 128);
    constexpr uint32_t HALF_BYTES = 32 * LW * 4, STAGE_BYTES = 2 * HALF_BYTES;
    constexpr int RAWB_OFS = 16 * QMV_SPITCH * 2;  // raw biases sit behind the raw scales
    const uint32_t cpk_s = sraw_s + QMV_RAW_BYTES;   // repacked constants of the current chunk

    // ── this warp's run of iterations ───────────────────────────────────────────────────
    // Two levels: the blocks take consecutive runs of the sequence whose lengths differ by at most
    // one (the first blk_r blocks hold blk_q + 1 iterations) and the warps of a block split the
    // block's run the same way.  The launch gives every block at least QMV_WARPS iterations unless
    // the grid is a single block, where surplus warps idle.  All of it is 32-bit arithmetic: the
    // launch refuses sequences of 2^30 iterations or more.
    const uint32_t blk_q = p.blk_q, blk_r = p.blk_r;
    // Run of part `i` when `len`-sized work is cut into parts of q or q + 1 (the first rm parts).
    auto part_lo = [](uint32_t i, uint32_t q, uint32_t rm) { return i * q + min(i, rm); };
    const uint32_t blk_lo = part_lo(blockIdx.x, blk_q, blk_r), blk_len = blk_q + (blockIdx.x < blk_r ? 1u : 0u);
    const uint32_t nw = min((uint32_t)QMV_WARPS, blk_len);
    const uint32_t wq = nw == QMV_WARPS ? blk_len / QMV_WARPS : 1u, wr = nw == QMV_WARPS ? blk_len % QMV_WARPS : 0u;
    const uint32_t lo = (uint32_t)warp < nw ? blk_lo + part_lo(warp, wq, wr) : 0u;
    const uint32_t hi = (uint32_t)warp < nw ? lo + wq + ((uint32_t)warp < wr ? 1u : 0u) : 0u;

    const uint32_t *wbase = p.w + wb * p.w_batch_stride + t * LW;
    const uint16_t *sc = (const uint16_t *)p.scales + wb * p.s_batch_stride;
    const uint16_t *bi = (const uint16_t *)p.biases + wb * p.s_batch_stride;
    __nv_bfloat16 *out = (__nv_bfloat16 *)p.y + b * p.M * p.N;
    // nvfp4 global scale: one value, or one per expert (quantized.rs:481-490, 700-712)
    const float gmul = U::FP && p.global ? (p.expert_global ? p.global[wb] : p.global[0]) / (448.0f * 6.0f) : 1.0f;

    const uint32_t sfast_dst = sraw_s + (lane >> 1) * (QMV_SPITCH * 2) + (lane & 1) * 16;
    // Copies the scales and biases of k-chunk `chunk` of `tile` into buffer `buf` (whole warp): two
    // lanes per row, each taking every other piece of the row's chunk.
    auto stage_scales = [&](int tile, int chunk, int buf) {
        const int rr = lane >> 1;
        const int64_t at0 = (int64_t)min(tile * 16 + rr, last_row) * row_groups + chunk * chunk_groups;
        if (U::FP) {
            // one scale byte per group, no biases: the two buffers share the whole per-warp area,
            // 16 rows of QMV_FPITCH bytes each
            const uint8_t *src = (const uint8_t *)p.scales + wb * p.s_batch_stride + at0;
            uint8_t *fd = reinterpret_cast<uint8_t *>(sraw) + buf * (16 * QMV_FPITCH) + rr * QMV_FPITCH;
            if (p.s_vec == 4) {
                for (int c = lane & 1; c < (chunk_groups >> 2); c += 2)
                    cp_async<4>((uint32_t)__cvta_generic_to_shared(fd + 4 * c), src + 4 * c);
            } else {
                for (int c = lane & 1; c < chunk_groups; c += 2) fd[c] = src[c];
            }
            return;
        }
        const uint16_t *ss = sc + at0, *bs = bi + at0;
        if (p.s_vec == 32) {  // the usual case, 16 groups per chunk in 16-byte pieces: one piece of each array per lane
            cp_async_at<16, 0, 0>(sfast_dst, ss + 8 * (lane & 1));
            cp_async_at<16, RAWB_OFS, 0>(sfast_dst, bs + 8 * (lane & 1));
            return;
        }
        uint16_t *sd = sraw + rr * QMV_SPITCH;  // (affine: one raw buffer, repacked before the next copy starts)
        uint16_t *bd = braw + rr * QMV_SPITCH;
        if (p.s_vec == 16) {  // 16-byte copies of 8 groups
            for (int c = lane & 1; c < (chunk_groups >> 3); c += 2) {
                cp_async<16>((uint32_t)__cvta_generic_to_shared(sd + 8 * c), ss + 8 * c);
                cp_async<16>((uint32_t)__cvta_generic_to_shared(bd + 8 * c), bs + 8 * c);
            }
        } else if (p.s_vec == 4) {  // 4-byte copies of 2 groups
            for (int c = lane & 1; c < (chunk_groups >> 1); c += 2) {
                cp_async<4>((uint32_t)__cvta_generic_to_shared(sd + 2 * c), ss + 2 * c);
                cp_async<4>((uint32_t)__cvta_generic_to_shared(bd + 2 * c), bs + 2 * c);
            }
        } else {
            for (int c = lane & 1; c < chunk_groups; c += 2) {
                sd[c] = ss[c];
                bd[c] = bs[c];
            }
        }
    };

    // Start of the run: the only divisions of the kernel outside tiles cut by a run boundary.
    const int tile0 = (int)(lo / (uint32_t)ipt), it_first = (int)(lo - (uint32_t)tile0 * (uint32_t)ipt);
    const int chunk0 = it_first / ci;

    // Prefetch cursor: the iteration whose words are copied next.
    uint32_t pf_left = hi - lo;      // iterations of the run not yet requested
    int pf_tile = tile0;
    int pf_wrap = ipt - it_first;    // iterations until the cursor enters the next tile
    const uint32_t *pf_a = nullptr, *pf_q = nullptr;
    auto pf_rows = [&](int it) {
        if constexpr (ROWMAJOR) {  // one pointer: this lane's half of row piece lane / 2
            pf_a = p.w + wb * p.w_batch_stride + (size_t)min(pf_tile * 16 + (lane >> 1), last_row) * row_words +
                   it * (4 * LW) + (lane & 1) * (HB / 4);
            return;
        }
        pf_a = wbase + (size_t)min(pf_tile * 16 + r, last_row) * row_words + it * (4 * LW);
        pf_q = wbase + (size_t)min(pf_tile * 16 + r + 8, last_row) * row_words + it * (4 * LW);
    };
    // The 16-byte copies of a 3-word-unit iteration: destination `dst` (this lane's place in the stage),
    // source pf_a + GOFS bytes.
    auto copy_row_parts = [&](uint32_t dst, auto sofs_c, auto gofs_c) {
        constexpr int SOFS = decltype(sofs_c)::value, GOFS = decltype(gofs_c)::value;
        static_for<PARTS>([&](auto k_) {
            constexpr int k = decltype(k_)::value;
            cp_async_at<16, SOFS + 16 * k, GOFS + 16 * k>(dst, pf_a);
        });
        if (extra_part) cp_async_at<16, SOFS + 32, GOFS + 32>(dst, pf_a);
    };
    // Issues the copies of one iteration into the stage at shared address `slot` and always commits
    // one group, so the group count seen by wait_group is the same for every lane and iteration.
    auto prefetch = [&](uint32_t slot) {
        if (pf_left != 0u) {
            if constexpr (ROWMAJOR) {
                // (`slot` is this lane's place for reading; its place for copying lies copy_s - ring_s further)
                copy_row_parts(slot + (copy_s - ring_s), std::integral_constant<int, 0>{}, std::integral_constant<int, 0>{});
            } else {
                static_for<CPL>([&](auto c_) {
                    constexpr int c = decltype(c_)::value;
                    cp_async_at<CW * 4, c * (32 * CW * 4), c * CW * 4>(slot, pf_a);
                    cp_async_at<CW * 4, HALF_BYTES + c * (32 * CW * 4), c * CW * 4>(slot, pf_q);
                });
            }
            pf_a += 4 * LW;
            pf_q += 4 * LW;
            pf_left--;
            if (--pf_wrap == 0) {
                pf_wrap = ipt;
                pf_tile++;
                pf_rows(0);
            }
        }
        cp_async_commit();
    };
    // The ring stage of an iteration is its index in the tile modulo the ring depth whenever tiles
    // and k-chunks are whole rounds of the ring (p.rounds): aligned rounds then know their stages at
    // compile time.
    const uint32_t first_stage = (uint32_t)it_first % QMV_STAGES;

    // Programmatic dependent launch: the next kernel of the stream may be scheduled from now on,
    // and this one starts copying weights (which no product writes) while the kernel before it is
    // still finishing; only then does it wait for that kernel's results.
    if (p.early_weights) {
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    } else {
        // the caller's stream may hold a kernel that writes these weights: nothing is read early
        asm volatile("griddepcontrol.wait;" ::: "memory");
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    }
    if (lo < hi) {
        stage_scales(tile0, chunk0, 0);
        pf_rows(it_first);
    }
#pragma unroll
    for (int st = 0; st < QMV_STAGES; st++) prefetch(ring_s + ((first_stage + st) % QMV_STAGES) * STAGE_BYTES);
    QMV_TIMELINE_MARK(1)
    if (p.early_weights)
        asm volatile("griddepcontrol.wait;" ::: "memory");  // activations, scratch and output belong to this kernel from here
    QMV_TIMELINE_MARK(2)
    // ── stage the activations once per block (the first weight copies are already in flight) ──
    {
        const uint16_t *x = (const uint16_t *)p.x + xb * p.x_batch_stride;
        const int blocks_per_row = (int)(row_words / UW);  // units (8-, 4-, 16- or 32-value blocks) per row
        for (int m = 0; m < p.M; m++) {
            const uint16_t *xrow_src = x + (int64_t)m * p.ldx;
            uint32_t *xrow_dst = xs + (size_t)m * xs_pitch;
            if (CODES == 8 && p.x_vec) {
                // eight values per unit (4-bit codes): the pairs (x0,x4) (x1,x5) (x2,x6) (x3,x7) come out
                // of one 16-byte load with four byte permutations and go back as one 16-byte store
                // (the loads of up to four units per thread are issued together: the block pays one
                // round trip to L2 for a row of 8192 values instead of four)
                constexpr int XB = 4;
                for (int blk0 = tid; blk0 < blocks_per_row; blk0 += XB * QMV_THREADS) {
                    uint4 in[XB];
#pragma unroll
                    for (int u = 0; u < XB; u++)
                        if (blk0 + u * QMV_THREADS < blocks_per_row)
                            in[u] = __ldcg(reinterpret_cast<const uint4 *>(xrow_src) + blk0 + u * QMV_THREADS);
#pragma unroll
                    for (int u = 0; u < XB; u++) {
                        const int blk = blk0 + u * QMV_THREADS;
                        if (blk < blocks_per_row) {
                            uint4 o;
                            o.x = __byte_perm(in[u].x, in[u].z, 0x5410); o.y = __byte_perm(in[u].x, in[u].z, 0x7632);
                            o.z = __byte_perm(in[u].y, in[u].w, 0x5410); o.w = __byte_perm(in[u].y, in[u].w, 0x7632);
                            const int it = blk / (4 * WPL), tt = (blk / WPL) & 3, j = blk % WPL;
                            *reinterpret_cast<uint4 *>(xrow_dst + (size_t)(((it * WPL + j) * 4 + tt) * XW)) = o;
                        }
                    }
                }
                continue;
            }
            for (int blk = tid; blk < blocks_per_row; blk += QMV_THREADS) {
                uint16_t in[CODES], outv[XW * 2];
                const uint16_t *src = xrow_src + (int64_t)blk * CODES;
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
                // unit `blk` of the row belongs to iteration blk / (4 WPL), lane t = (blk / WPL) % 4, unit j = blk % WPL
                const int it = blk / (4 * WPL), tt = (blk / WPL) & 3, j = blk % WPL;
                uint32_t *dst = xrow_dst + (size_t)(((it * WPL + j) * 4 + tt) * XW);
#pragma unroll
                for (int v = 0; v < XW; v++) dst[v] = (uint32_t)outv[2 * v] | ((uint32_t)outv[2 * v + 1] << 16);
            }
        }
        for (int i = tid; i < ZERO_WORDS; i += QMV_THREADS) zero[i] = 0u;
        if (tid < QMV_WARPS) lcount[tid] = 0u;
        if (p.peer) {
            // fused collectives: the ranks' region addresses and this product's sequence number (the
            // count of fused products this rank has finished, plus one: every rank runs the same
            // sequence of them, so the numbers agree across ranks without any exchange)
            if (tid < 16) reinterpret_cast<void **>(lcount + QMV_WARPS + 4)[tid] = p.peer->base[tid];
            if (tid == 0) lcount[QMV_WARPS + 1] = __ldcg(static_cast<const uint32_t *>(p.peer->base[p.peer_rank]) + 16) + 1u;
        }
    }
    __syncthreads();  // activations staged
    QMV_TIMELINE_MARK(3)

    const bool xrow = r < p.M;
    const uint32_t x_it_bytes = xrow ? X_IT_WORDS * 4 : 0;  // bytes per iteration in xs (0: stay on the zero page)
    const uint32_t xbase_s = (uint32_t)__cvta_generic_to_shared(xrow ? xs + (size_t)r * xs_pitch + t * XW : zero + t * XW);
    int seg_count = 0;   // segments started so far (buffer parity)
    int prev_iters = 0;  // iterations of the previous segment
    uint32_t rs = ring_s + first_stage * STAGE_BYTES;  // this lane's slot in the ring stage consumed next
    const uint32_t rs_end = ring_s + QMV_STAGES * STAGE_BYTES;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};  // rows r / r+8 x activation rows 2t / 2t+1
    float acd[4] = {0.f, 0.f, 0.f, 0.f};  // second accumulator: halves the MMA dependency chain
    // per-segment state of the iteration body
    uint32_t kofs = 0;    // k offset of this lane's words inside the chunk
    uint32_t srow_s = 0;  // staged scale of (row r, group 0) of the segment's buffer; row r + 8, the biases
                          // and the group are offsets from it
    uint32_t xa = 0;      // this lane's activation words of the current iteration

    // One iteration.  J >= 0: the iteration is number J of an aligned round of QMV_STAGES whose ring
    // stages, activation words and weight addresses are compile-time offsets from round-invariant
    // registers, and whose copies need no end-of-run or end-of-tile checks; J < 0: anywhere, with
    // every position kept in registers.
    auto iteration = [&](auto stage_c, auto copy_c) {
        constexpr int J = decltype(stage_c)::value;
        constexpr bool FIX = J >= 0;
        constexpr bool COPY = decltype(copy_c)::value;  // (rounds only) refill the stage; false once the run's last words are requested
        constexpr int SO = FIX ? J * (int)STAGE_BYTES : 0;   // offset of the stage from the base address
        constexpr int XO = FIX ? J * X_IT_WORDS * 4 : 0;     // offset of the iteration's activations
        const uint32_t sb = FIX ? ring_s : rs;
        cp_async_wait<QMV_STAGES - 1>();  // the oldest group, this iteration's words, has landed
        uint32_t wa_[LW], wq_[LW];
        if constexpr (LW == 3) {  // lane 4 r + t: words 3 (4 r + t) .. + 2 of the half, conflict-free word by word
            static_for<3>([&](auto c_) {
                constexpr int c = decltype(c_)::value;
                wa_[c] = lds32<SO + c * 4>(sb);
                wq_[c] = lds32<SO + (int)HALF_BYTES + c * 4>(sb);
            });
        } else if constexpr (LW == 6 && UW == 3) {  // 24 bytes per lane: three 8-byte loads
            static_for<3>([&](auto c_) {
                constexpr int c = decltype(c_)::value;
                const uint2 a = lds64<SO + c * 8>(sb), q = lds64<SO + (int)HALF_BYTES + c * 8>(sb);
                wa_[2 * c] = a.x; wa_[2 * c + 1] = a.y;
                wq_[2 * c] = q.x; wq_[2 * c + 1] = q.y;
            });
        } else if constexpr (WPL == 8) {
            static_for<2>([&](auto c_) {
                constexpr int c = decltype(c_)::value;
                uint4 a = lds128<SO + c * 512>(sb);
                uint4 q = lds128<SO + (int)HALF_BYTES + c * 512>(sb);
                wa_[(4 * c) % WPL] = a.x; wa_[(4 * c + 1) % WPL] = a.y; wa_[(4 * c + 2) % WPL] = a.z; wa_[(4 * c + 3) % WPL] = a.w;
                wq_[(4 * c) % WPL] = q.x; wq_[(4 * c + 1) % WPL] = q.y; wq_[(4 * c + 2) % WPL] = q.z; wq_[(4 * c + 3) % WPL] = q.w;
            });
        } else if constexpr (WPL == 4) {
            uint4 a = lds128<SO>(sb), q = lds128<SO + (int)HALF_BYTES>(sb);
            wa_[0] = a.x; wa_[1 % WPL] = a.y; wa_[2 % WPL] = a.z; wa_[3 % WPL] = a.w;
            wq_[0] = q.x; wq_[1 % WPL] = q.y; wq_[2 % WPL] = q.z; wq_[3 % WPL] = q.w;
        } else if constexpr (WPL == 2) {
            uint2 a = lds64<SO>(sb), q = lds64<SO + (int)HALF_BYTES>(sb);
            wa_[0] = a.x; wa_[1 % WPL] = a.y;
            wq_[0] = q.x; wq_[1 % WPL] = q.y;
        } else {
            wa_[0] = lds32<SO>(sb);
            wq_[0] = lds32<SO + (int)HALF_BYTES>(sb);
        }
        const uint32_t g = (kofs + (FIX ? J * IK : 0)) >> p.gs_shift;
        if (!FIX) kofs += IK;
        GroupConsts ga, gq, ga1, gq1;  // (ga1, gq1: the second group of a lane's words, nvfp4 only)
        if constexpr (U::FP != 0) {
            const uint32_t fa = srow_s + g;
            ga.s2 = fp4_scale2(lds_u8<0>(fa), U::FP == 1); gq.s2 = fp4_scale2(lds_u8<8 * QMV_FPITCH>(fa), U::FP == 1);
            ga.b2 = gq.b2 = ga.ns2 = gq.ns2 = 0u;
            ga1 = ga; gq1 = gq;
            if (U::FP == 3 && WPL * CODES > 16) {
                ga1.s2 = fp4_scale2(lds_u8<1>(fa), false);
                gq1.s2 = fp4_scale2(lds_u8<8 * QMV_FPITCH + 1>(fa), false);
            }
        } else {
            const uint32_t ca = srow_s + g * QMV_PKPITCH;
            const uint2 ea = lds64<0>(ca), eq = lds64<8 * 8>(ca);
            ga.s2 = ea.x; ga.b2 = ea.y;
            gq.s2 = eq.x; gq.b2 = eq.y;
            ga.ns2 = bf2_mul(ga.s2, 0xC300C300u);  // -128 s, exact
            gq.ns2 = bf2_mul(gq.s2, 0xC300C300u);
            ga1 = ga; gq1 = gq;
        }
        static_for<WPL>([&](auto j_) {
            constexpr int j = decltype(j_)::value;
            uint32_t ra[AREGS], rq[AREGS], xr[XW];
            constexpr bool second = U::FP == 3 && j * CODES >= 16;  // nvfp4: 16 values per scale
            U::run(&wa_[j * UW], second ? ga1 : ga, ra);
            U::run(&wq_[j * UW], second ? gq1 : gq, rq);
            if constexpr (XW == 2) {
                uint2 q = lds64<XO + j * (4 * XW * 4)>(xa);
                xr[0] = q.x; xr[1] = q.y;
            } else {
                static_for<XW / 4>([&](auto v_) {
                    constexpr int v = 4 * decltype(v_)::value;
                    uint4 q = lds128<XO + j * (4 * XW * 4) + v * 4>(xa);
                    xr[v] = q.x; xr[v + 1] = q.y; xr[v + 2] = q.z; xr[v + 3] = q.w;
                });
            }
#pragma unroll
            for (int h = 0; h < AREGS / 2; h++) {
                if ((j * (AREGS / 2) + h) & 1)
                    mma_bf16_16816(acd, ra[2 * h], rq[2 * h], ra[2 * h + 1], rq[2 * h + 1], xr[2 * h], xr[2 * h + 1]);
                else
                    mma_bf16_16816(acc, ra[2 * h], rq[2 * h], ra[2 * h + 1], rq[2 * h + 1], xr[2 * h], xr[2 * h + 1]);
            }
        });
        // Refill the slot just consumed (its words are in registers and already used).
        if constexpr (FIX) {
            if constexpr (COPY && ROWMAJOR) {
                copy_row_parts(copy_s, std::integral_constant<int, SO>{}, std::integral_constant<int, J * 4 * LW * 4>{});
            } else if constexpr (COPY) {
                static_for<CPL>([&](auto c_) {
                    constexpr int c = decltype(c_)::value;
                    cp_async_at<CW * 4, SO + c * (32 * CW * 4), (J * 4 * LW + c * CW) * 4>(ring_s, pf_a);
                    cp_async_at<CW * 4, SO + (int)HALF_BYTES + c * (32 * CW * 4), (J * 4 * LW + c * CW) * 4>(ring_s, pf_q);
                });
            }
            cp_async_commit();
        } else {
            xa += x_it_bytes;
            prefetch(rs);
            rs += STAGE_BYTES;
            if (rs == rs_end) rs = ring_s;
        }
    };
    const bool rounds = p.rounds != 0;

    int tile = tile0, it0 = it_first, chunk = chunk0;  // position of f in the sequence, kept without divisions
    for (uint32_t f = lo; f < hi;) {
        // Segment: the part of one k-chunk of one tile that lies in [f, hi).
        const int cend = (chunk + 1) * ci;
        const int it1 = (int)min((uint32_t)cend, hi - f + (uint32_t)it0);
        const uint32_t f1 = f + (uint32_t)(it1 - it0);
        const int seg_buf = seg_count & 1;
        // wait_group in the loop below covers a copy once QMV_STAGES groups were committed after it;
        // a shorter previous segment (or the very first one) needs an explicit wait.  Then the
        // copies of all lanes are made visible across the warp.
        if (prev_iters <= QMV_STAGES) cp_async_wait<0>();
        __syncwarp();
        if constexpr (U::FP == 0) {
            // Repack this chunk's raw scales and biases: lane (row rr, half hh) turns eight groups of its
            // row into the pairs {s, s}, {b, b} at [group][row]; every (row, group) is then one 8-byte
            // load per iteration instead of two 2-byte loads and two duplications.
            const int rr = lane >> 1, hh = lane & 1;
            const uint32_t raw = sraw_s + rr * (QMV_SPITCH * 2) + hh * 16;
            const uint4 sv = lds128<0>(raw), bv = lds128<RAWB_OFS>(raw);
            const uint32_t sw[4] = {sv.x, sv.y, sv.z, sv.w}, bw[4] = {bv.x, bv.y, bv.z, bv.w};
            const uint32_t dst = cpk_s + hh * (8 * QMV_PKPITCH) + rr * 8;
            static_for<8>([&](auto i_) {
                constexpr int i = decltype(i_)::value;
                constexpr uint32_t sel = (i & 1) ? 0x3232u : 0x1010u;
                sts64<i * QMV_PKPITCH>(dst, __byte_perm(sw[i >> 1], 0u, sel), __byte_perm(bw[i >> 1], 0u, sel));
            });
            __syncwarp();  // the constants are complete and the raw buffer is free
        }
        // The next segment's scales start their way into the buffer this one no longer needs.
        if (f1 < hi) {  // the run goes on, so this segment ends with its chunk
            const bool wrap = it1 == ipt;
            stage_scales(wrap ? tile + 1 : tile, wrap ? 0 : chunk + 1, (seg_count + 1) & 1);
        }
        prev_iters = it1 - it0;
        seg_count++;
        kofs = (uint32_t)((it0 - chunk * ci) * IK + t * (WPL * CODES));
        srow_s = U::FP ? sraw_s + seg_buf * (16 * QMV_FPITCH) + r * QMV_FPITCH : cpk_s + r * 8;
        xa = xbase_s + (uint32_t)it0 * x_it_bytes;
        int it = it0;
        while (it < it1) {
            // An aligned round: QMV_STAGES iterations that start at a multiple of the ring depth and
            // whose copies (the QMV_STAGES iterations behind them) all lie inside the run; the cursor
            // can only reach the end of its tile after the last of them.
            if (QMV_STAGES == 4 && rounds && (it & 3) == 0 && it + 4 <= it1 && (pf_left >= 4u || pf_left == 0u)) {
                if (pf_left != 0u) {
                    static_for<4>([&](auto j_) { iteration(j_, std::true_type{}); });
                    pf_a += 4 * 4 * LW;
                    pf_q += 4 * 4 * LW;
                    pf_left -= 4u;
                    pf_wrap -= 4;
                    if (pf_wrap == 0) {
                        pf_wrap = ipt;
                        pf_tile++;
                        pf_rows(0);
                    }
                } else {
                    static_for<4>([&](auto j_) { iteration(j_, std::false_type{}); });
                }
                it += 4;
                kofs += 4 * IK;
                xa += 4 * x_it_bytes;
            } else {
                iteration(std::integral_constant<int, -1>{}, std::true_type{});
                it++;
            }
        }
        f = f1;
        if (it1 != ipt && f1 != hi) {  // the tile goes on in the next k-chunk
            it0 = it1;
            chunk++;
            continue;
        }
        const int done_tile = tile;
        if (it1 == ipt) {
            tile++;
            it0 = 0;
            chunk = 0;
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
        if (!store) {
            QmvCut c;
            c.lo = lo; c.hi = hi; c.blk_lo = blk_lo; c.blk_len = blk_len; c.wq = wq; c.wr = wr;
            c.blk_q = blk_q; c.blk_r = blk_r; c.t_lo = t_lo; c.t_hi = t_hi;
            c.warp = warp; c.lane = lane; c.first_tile = done_tile == tile0 ? 1 : 0;
            c.max_parts = p.max_parts; c.lpart = lpart; c.lcount = lcount;
            c.partials = p.partials; c.counters = p.counters; c.slot0 = b * gridDim.x;
            float4 vv = make_float4(v[0], v[1], v[2], v[3]);
            store = qmv_meet_partials(c, vv);
            v[0] = vv.x; v[1] = vv.y; v[2] = vv.z; v[3] = vv.w;
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
            // Fused collective.  Every result (gather: the rounded bfloat16; all-sum: this rank's float32
            // partial sum) travels as one 8-byte packet {value, sequence number} into the same slot of
            // every rank's packet area: an aligned 8-byte store arrives whole, so a reader that sees
            // the product's sequence number has the value with it -- no fence, no flag, and nothing
            // waits for this rank's other blocks.  Two areas alternate with the sequence number's
            // parity, so the next product on the same offsets never lands on packets still being read.
            const uint32_t seq = lcount[QMV_WARPS + 1];
            char *const *bases = reinterpret_cast<char *const *>(lcount + QMV_WARPS + 4);
            const size_t per = (size_t)p.M * p.N;  // values per rank
            const size_t area = p.peer_ll_offset + (size_t)(seq & 1u) * ((size_t)p.peer_size * per * 8);
            uint16_t *own_out = reinterpret_cast<uint16_t *>(bases[p.peer_rank] + p.peer_out_offset) + (size_t)p.peer_rank * per;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int row = n0 + r + (i >> 1) * 8, col = 2 * t + (i & 1);
                if (col < p.M && row <= last_row) {
                    const size_t e = (size_t)col * p.N + row;
                    uint32_t data;
                    if (p.peer_mode == 1) {  // gather: this rank's own slot is written directly
                        const __nv_bfloat16 h = __float2bfloat16_rn(v[i]);
                        data = (uint32_t)__bfloat16_as_ushort(h);
                        own_out[e] = (uint16_t)data;
                    } else {
                        data = __float_as_uint(v[i]);
                    }
                    const size_t slot = area + ((size_t)p.peer_rank * per + e) * 8;
                    for (int rk = 0; rk < p.peer_size; rk++) {
                        if (p.peer_mode == 1 && rk == p.peer_rank) continue;
                        asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(bases[rk] + slot), "r"(data), "r"(seq) : "memory");
                    }
                }
            }
        }
    }
    QMV_TIMELINE_END(lo < hi)
    cp_async_wait<0>();
    if (p.peer) {
        // Second half of the fused collective: all threads of the grid share the packets this rank
        // receives.  A thread waits (bounded: about a second, then the error word says so) until its
        // packet carries this product's sequence number and consumes it -- gather: the value goes
        // into the gathered buffer; all-sum: the ranks' partial sums of one result are added in rank
        // order, rounded once and stored, identically on every rank.  When the kernel ends the
        // result is complete on this rank, so the next kernel of the stream needs no wait of its own.
        const uint32_t seq = lcount[QMV_WARPS + 1];
        char *const *bases = reinterpret_cast<char *const *>(lcount + QMV_WARPS + 4);
        char *own = bases[p.peer_rank];
        const size_t per = (size_t)p.M * p.N;
        const char *area = own + p.peer_ll_offset + (size_t)(seq & 1u) * ((size_t)p.peer_size * per * 8);
        const size_t gtid = (size_t)blockIdx.x * QMV_THREADS + tid, gthreads = (size_t)gridDim.x * QMV_THREADS;
        bool late = false;
        auto packet = [&](size_t index, uint32_t &data) {
            const char *at = area + index * 8;
            uint32_t s2 = 0;
            for (uint32_t spins = 0; spins < (1u << 20); spins++) {
                asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(data), "=r"(s2) : "l"(at) : "memory");
                if (s2 == seq) return true;
            }
            return false;
        };
        if (p.peer_mode == 1) {
            uint16_t *gathered = reinterpret_cast<uint16_t *>(own + p.peer_out_offset);
            for (size_t i = gtid; i < (size_t)p.peer_size * per; i += gthreads) {
                if (i / per == (size_t)p.peer_rank) continue;
                uint32_t data;
                if (packet(i, data)) gathered[i] = (uint16_t)data;
                else late = true;
            }
        } else {
            __nv_bfloat16 *y = (__nv_bfloat16 *)p.y;
            for (size_t e = gtid; e < per; e += gthreads) {
                float sum = 0.f;
                bool ok = true;
                for (int rk = 0; rk < p.peer_size; rk++) {
                    uint32_t data;
                    if (packet((size_t)rk * per + e, data)) sum += __uint_as_float(data);
                    else ok = false;
                }
                if (ok) y[e] = __float2bfloat16_rn(sum);
                else late = true;
            }
        }
        if (late && p.error) *p.error = 2;
        // the count of finished fused products advances once the last block is through
        __syncthreads();
        if (tid == 0) {
            uint32_t *head = reinterpret_cast<uint32_t *>(own);
            __threadfence();
            if (atomicAdd(head + 17, 1u) == gridDim.x * gridDim.z - 1) {
                head[17] = 0u;
                __stcg(head + 16, seq);
                __stcg(head + p.peer_rank, seq);
            }
        }
    }
}

// ── host side ──────────────────────────────────────────────────────────────────────────

// A unit is the smallest run of words that holds whole codes: one word, or three for 3 and 6 bits.
// (`bits` below is the kernel's kind: the affine bit width, or 40 = mxfp4, 41 = nvfp4, 42 = mxfp8.)
static bool kind_fp(int bits) { return bits == 40 || bits == 41 || bits == 42; }
static int code_bits(int bits) { return bits == 42 ? 8 : kind_fp(bits) ? 4 : bits; }
static int unit_words(int bits) { return bits == 3 || bits == 6 ? 3 : 1; }
static int codes_per_word(int bits) { return unit_words(bits) * 32 / code_bits(bits); }  // codes per unit
int qmv_kind(int32_t mode, int32_t bits) {
    if (mode == NVC_AFFINE) return bits;
    if (mode == NVC_MXFP4 && bits == 4) return 40;
    if (mode == NVC_NVFP4 && bits == 4) return 41;
    if (mode == NVC_MXFP8 && bits == 8) return 42;
    return 0;
}

// Words per lane per iteration: the widest vector load, up to four words, whose 4-lane span divides
// K.  (Eight words, two 16-byte copies, execute fewer instructions per weight but were measured to
// issue slower on the B200 than four.)
static int wpl_for(int bits, int gs, int64_t K) {
    if (bits != 2 && bits != 3 && bits != 4 && bits != 6 && bits != 8 && !kind_fp(bits)) return 0;
    const int codes = codes_per_word(bits);
    const int cap = 4;
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
    return (size_t)(M * (K / codes * xw + 16) + qmv_zero_words(wpl, xw) + QMV_WARPS * (QMV_SCALE_AREA / 4) +
                    qmv_stages(wpl) * 2 * QMV_THREADS * lw + QMV_WARPS * 2 * 128 + QMV_WARPS + 4 + 32) * 4 + 16;
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
    const int cw = unit_words(bits) == 3 ? 4 : wpl == 8 ? 4 : wpl;  // words per asynchronous copy (3-word units: 16-byte parts of a row)
    if (row_words % cw != 0 || w_batch_stride % cw != 0 || ((uintptr_t)w % (4 * cw)) != 0) return false;
    if (((N + 15) / 16) * (K / (4 * wpl * codes_per_word(bits))) >= (int64_t)1 << 30) return false;  // 32-bit iteration counts
    return qmv_smem((int)M, K, bits, wpl) <= 220 * 1024;  // all activations are staged in shared memory
}

// The opt-in to more than 48 KB of dynamic shared memory is a per-device attribute of each kernel
// instantiation: the largest size set so far is kept per device ordinal.
constexpr int QMV_MAX_DEVICES = 64;
static std::mutex g_qmv_cfg_mu;

template <int BITS, int WPL>
static int32_t launch_qmv_cfg(nvc_device *dev, QmvParams &p, dim3 grid, size_t smem) {
    auto kernel = qmv_affine_kernel<BITS, WPL>;
    static size_t configured[QMV_MAX_DEVICES] = {};
    if (dev->ordinal < 0 || dev->ordinal >= QMV_MAX_DEVICES)
        return set_error(NVC_ERR_UNSUPPORTED, "qmv: device ordinal %d", dev->ordinal);
    if (smem > 48 * 1024) {
        std::lock_guard<std::mutex> g(g_qmv_cfg_mu);
        if (smem > configured[dev->ordinal]) {
            NVC_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            configured[dev->ordinal] = smem;
        }
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
    // On a stream adopted from the caller the kernel before this one may be anybody's, including one
    // that produces these weights: nothing is read ahead of it there.
    p.early_weights = dev->stream == dev->own_stream ? 1 : 0;
    NVC_CUDA(cudaLaunchKernelEx(&cfg, kernel, p));
    return check_launch(dev, "qmv_affine_kernel");
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
        else if (al % 16 == 0 && p.s_batch_stride % 8 == 0 && rg % 8 == 0 && cg % 8 == 0) p.s_vec = cg == 16 ? 32 : 16;
        else if (al % 4 == 0 && p.s_batch_stride % 2 == 0 && rg % 2 == 0 && cg % 2 == 0) p.s_vec = 4;
        else p.s_vec = 0;
    }
    const size_t smem = qmv_smem(p.M, p.K, bits, wpl);
    // Blocks: as many as stay resident (two per multiprocessor while shared memory allows), but
    // no more than give every warp a few iterations.
    // (each block also takes 1 KB of shared memory the system reserves)
    // Row-exact products (nvc_set_row_exact) are cut as one row of one batch would be, whatever M and the
    // number of batches are: the cuts decide the order of a row's float32 sums, and every row must get the
    // bits of its one-row product.  (Blocks beyond the resident ones queue; none waits for another.)
    const size_t plan_smem = dev->row_exact ? qmv_smem(1, p.K, bits, wpl) : smem;
    const int64_t plan_batch = dev->row_exact ? 1 : batch;
    int64_t per_sm = (int64_t)(227 * 1024) / (int64_t)(plan_smem + 1024);
    if (per_sm > QMV_BLOCKS_PER_SM) per_sm = QMV_BLOCKS_PER_SM;
    if (per_sm < 1) per_sm = 1;
    int64_t blocks = per_sm * dev->prop.multiProcessorCount / plan_batch;
    const int64_t min_iters = 4;
    const int64_t useful = (total + QMV_WARPS * min_iters - 1) / (QMV_WARPS * min_iters);
    if (blocks > useful) blocks = useful;
    if (blocks > 1) {
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
    p.row_groups = (int32_t)(p.K / p.gs);
    p.row_words = (uint32_t)(p.K * code_bits(bits) / 32);
    p.ipt = (int32_t)ipt;
    p.ci = (int32_t)(chunk / ik);
    p.chunk_groups = (int32_t)(chunk / p.gs);
    p.tiles = (int32_t)tiles;
    p.rounds = (ipt % 4 == 0 && p.ci % 4 == 0) ? 1 : 0;
    p.xs_pitch = (int32_t)(p.K / codes * (codes / 2) + 16);
    if (!p.rhs) p.experts = p.x_batches = 0;
    // Only tiles cut by a block boundary use global scratch, and such a tile is named by its first
    // block: one slot of max_parts partial tiles and one counter per (batch, block).
    const size_t partial_bytes = (size_t)blocks * batch * p.max_parts * 128 * sizeof(float);
    if (fixed) {
        // Scratch of fixed capacity provided by the caller of this function: nothing is allocated.
        if (partial_bytes > fixed->partial_bytes || (size_t)(blocks * batch) > fixed->counters_len)
            return set_error(NVC_ERR_UNSUPPORTED,
                             "qmv: this product needs %zu bytes of partial sums and %lld counters; the fixed scratch holds "
                             "%zu bytes and %zu counters", partial_bytes, (long long)(blocks * batch), fixed->partial_bytes,
                             fixed->counters_len);
        p.partials = fixed->partials;
        p.counters = fixed->counters;
    } else {
        void *scratch = nullptr;
        NVC_TRY(ensure_scratch(dev, partial_bytes, &scratch));
        p.partials = (float *)scratch;
        NVC_TRY(ensure_counters(dev, (size_t)(blocks * batch), &p.counters));
    }
    dim3 grid((unsigned)blocks, 1, (unsigned)batch);
#define NVC_QMV(B, W) if (bits == B && wpl == W) return launch_qmv_cfg<B, W>(dev, p, grid, smem);
    NVC_QMV(4, 1) NVC_QMV(4, 2) NVC_QMV(4, 4) NVC_QMV(4, 8) NVC_QMV(8, 1) NVC_QMV(8, 2) NVC_QMV(8, 4) NVC_QMV(8, 8)
    NVC_QMV(2, 1) NVC_QMV(2, 2) NVC_QMV(3, 1) NVC_QMV(6, 1) NVC_QMV(6, 2)
    NVC_QMV(40, 1) NVC_QMV(40, 2) NVC_QMV(40, 4) NVC_QMV(41, 1) NVC_QMV(41, 2) NVC_QMV(41, 4)
    NVC_QMV(42, 1) NVC_QMV(42, 2) NVC_QMV(42, 4)
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
constexpr size_t NOALLOC_COUNTERS = 16384;  // one per block of a launch (at most two blocks per multiprocessor)
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
    // The array keeps whatever the last call left; the counters must start at zero.  One counter per
    // block of the launch, and a grid never has more than two blocks per multiprocessor.
    const size_t used = (size_t)2 * dev->prop.multiProcessorCount;
    if (used > NOALLOC_COUNTERS)
        return set_error(NVC_ERR_UNSUPPORTED, "quantized_matmul (no-alloc): %d multiprocessors exceed the fixed scratch",
                         dev->prop.multiProcessorCount);
    NVC_CUDA(cudaMemsetAsync(fixed.counters, 0, used * sizeof(uint32_t), dev->stream));
    QmvParams p{};
    p.x = x; p.w = w; p.scales = scales; p.biases = biases; p.lhs = nullptr; p.rhs = nullptr; p.y = y;
    p.N = N; p.K = K; p.ldx = K;
    p.x_batch_stride = 0; p.w_batch_stride = 0; p.s_batch_stride = 0;
    p.M = (int32_t)M; p.gs = q->group_size;
    p.x_vec = ((uintptr_t)x % 16 == 0) && (K % 8 == 0);
    return launch_qmv_affine(dev, q->bits, p, 1, &fixed);
}

#ifdef NUVEC_TIMELINE
// Diagnostic build only.  Reset: every minimum to the largest value, every maximum to 0, record 0 next.
extern "C" int32_t nvc_debug_timeline_reset(void) {
    static unsigned long long init[nvc::TIMELINE_RECORDS][2 * nvc::TIMELINE_POINTS];
    for (auto &rec : init)
        for (int k = 0; k < 2 * nvc::TIMELINE_POINTS; k++) rec[k] = (k & 1) ? 0ull : ~0ull;
    const unsigned int zero = 0;
    if (cudaDeviceSynchronize() != cudaSuccess || cudaMemcpyToSymbol(nvc::g_timeline, init, sizeof init) != cudaSuccess ||
        cudaMemcpyToSymbol(nvc::g_timeline_at, &zero, sizeof zero) != cudaSuccess ||
        cudaMemcpyToSymbol(nvc::g_timeline_done, &zero, sizeof zero) != cudaSuccess)
        return NVC_ERR_DRIVER;
    return cudaDeviceSynchronize() == cudaSuccess ? NVC_OK : NVC_ERR_DRIVER;
}
// Copies the first `records` records ({min, max} nanoseconds of the six points each) to `out` and
// returns how many launches have been recorded since the reset (negative on error).
extern "C" int32_t nvc_debug_timeline_read(unsigned long long *out, int32_t records) {
    unsigned int launches = 0;
    if (records > nvc::TIMELINE_RECORDS) records = nvc::TIMELINE_RECORDS;
    if (cudaDeviceSynchronize() != cudaSuccess ||
        cudaMemcpyFromSymbol(&launches, nvc::g_timeline_at, sizeof launches) != cudaSuccess ||
        cudaMemcpyFromSymbol(out, nvc::g_timeline, sizeof(unsigned long long) * 2 * nvc::TIMELINE_POINTS * (size_t)records) != cudaSuccess)
        return -1;
    return (int32_t)launches;
}
#endif
