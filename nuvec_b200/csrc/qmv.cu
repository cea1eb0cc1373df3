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
//    by up to 8 activation rows per instruction.  Codes enter as the bfloat16 number
//    128 + code (one LOP3 per two codes: the code bits are ORed into the mantissa of 128.0),
//    per-group scale and bias are applied to the float32 group sums:
//        sum_k x*(s*c + b) = s * sum_k x*(128 + c)  +  (b - 128 s) * sum_k x.
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

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t orv) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;\n" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));  // (a & mask) | orv
    return r;
}

// Streaming loads of packed words: read-only path, no L1 allocation (each word is used once).
__device__ __forceinline__ void ldg_stream(uint32_t (&v)[1], const uint32_t *p) {
    asm volatile("ld.global.nc.L1::no_allocate.b32 %0, [%1];\n" : "=r"(v[0]) : "l"(p));
}
__device__ __forceinline__ void ldg_stream(uint32_t (&v)[2], const uint32_t *p) {
    asm volatile("ld.global.nc.L1::no_allocate.v2.b32 {%0,%1}, [%2];\n" : "=r"(v[0]), "=r"(v[1]) : "l"(p));
}
__device__ __forceinline__ void ldg_stream(uint32_t (&v)[4], const uint32_t *p) {
    asm volatile("ld.global.nc.L1::no_allocate.v4.b32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]) : "l"(p));
}

template <int BITS> struct Unpack;
// 4 bits: register i holds codes (i, i+4) of the word as the bf16 pair (128 + c_i, 128 + c_{i+4}).
template <> struct Unpack<4> {
    static constexpr int REGS = 4;      // bf16x2 registers per word
    static constexpr int CODES = 8;     // codes per word
    static constexpr int XREGS = 4;     // activation registers per word (bf16x2 each)
    static constexpr float OFFSET = 128.0f;  // sum of the slot weights of one k, times 128
    static __device__ __forceinline__ void run(uint32_t w, uint32_t (&r)[4]) {
#pragma unroll
        for (int i = 0; i < 4; i++) r[i] = lop3_and_or(w >> (4 * i), 0x000F000Fu, 0x43004300u);
    }
    // Activation order matching run(): pairs (x0,x4) (x1,x5) (x2,x6) (x3,x7).
    static __device__ __forceinline__ void permute(const __nv_bfloat16 *x, __nv_bfloat16 *out) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            out[2 * i] = x[i];
            out[2 * i + 1] = x[i + 4];
        }
    }
};
// 8 bits: each byte is split in its nibbles; a k-value occupies two MMA slots, the high nibble
// meeting 16 * x.  Registers: (lo0,lo2) (hi0,hi2) (lo1,lo3) (hi1,hi3).
template <> struct Unpack<8> {
    static constexpr int REGS = 4;
    static constexpr int CODES = 4;
    static constexpr int XREGS = 4;
    static constexpr float OFFSET = 128.0f * 17.0f;
    static __device__ __forceinline__ void run(uint32_t w, uint32_t (&r)[4]) {
#pragma unroll
        for (int i = 0; i < 4; i++) r[i] = lop3_and_or(w >> (4 * i), 0x000F000Fu, 0x43004300u);
    }
    static __device__ __forceinline__ void permute(const __nv_bfloat16 *x, __nv_bfloat16 *out) {
        const float f[4] = {__bfloat162float(x[0]), __bfloat162float(x[1]), __bfloat162float(x[2]), __bfloat162float(x[3])};
        out[0] = x[0]; out[1] = x[2];
        out[2] = __float2bfloat16_rn(16.0f * f[0]); out[3] = __float2bfloat16_rn(16.0f * f[2]);
        out[4] = x[1]; out[5] = x[3];
        out[6] = __float2bfloat16_rn(16.0f * f[1]); out[7] = __float2bfloat16_rn(16.0f * f[3]);
    }
};
// 2 bits: register i holds codes (i, i+8).
template <> struct Unpack<2> {
    static constexpr int REGS = 8;
    static constexpr int CODES = 16;
    static constexpr int XREGS = 8;
    static constexpr float OFFSET = 128.0f;
    static __device__ __forceinline__ void run(uint32_t w, uint32_t (&r)[8]) {
#pragma unroll
        for (int i = 0; i < 8; i++) r[i] = lop3_and_or(w >> (2 * i), 0x00030003u, 0x43004300u);
    }
    static __device__ __forceinline__ void permute(const __nv_bfloat16 *x, __nv_bfloat16 *out) {
#pragma unroll
        for (int i = 0; i < 8; i++) {
            out[2 * i] = x[i];
            out[2 * i + 1] = x[i + 8];
        }
    }
};

constexpr int QMV_WARPS = 8;
constexpr int QMV_UNROLL = 4;  // iterations whose loads are issued together

// Shared memory of one block:
//   xs   [M][kr / CODES * XREGS] u32   permuted activations of the block's k-range (+4 pad words per row)
//   xsum [8][groups] f32               per-group sums of x (rows >= M are zero)
//   sb   [16][groups] u32              (scale, bias) bf16 pairs of the block's 16 weight rows
//   red  [QMV_WARPS][128] f32          cross-warp reduction
template <int BITS, int WPL>
__global__ void __launch_bounds__(QMV_WARPS * 32) qmv_affine_kernel(QmvParams p) {
    using U = Unpack<BITS>;
    constexpr int CODES = U::CODES, REGS = U::REGS, XREGS = U::XREGS;
    constexpr int IK = 4 * WPL * CODES;  // k-values per iteration (one quad covers them)
    extern __shared__ __align__(16) uint32_t smem[];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int r = lane >> 2, t = lane & 3;
    const int64_t b = blockIdx.z;
    int64_t xb = b, wb = b;
    if (p.rhs) {
        wb = p.rhs[b];
        xb = p.lhs ? p.lhs[b] : b;
    }
    const int64_t n0 = (int64_t)blockIdx.x * 16;
    const int ks = blockIdx.y;
    const int64_t k0 = (int64_t)ks * p.kr;
    const int kr = (int)min((int64_t)p.kr, p.K - k0);  // multiple of the group size
    const int groups = kr / p.gs;
    const int g0 = (int)(k0 / p.gs);
    const int row_groups = (int)(p.K / p.gs);
    const int64_t row_words = p.K * BITS / 32;

    const int xs_pitch = p.kr / CODES * XREGS + 4;  // words
    uint32_t *xs = smem;
    float *xsum = (float *)(xs + (size_t)p.M * xs_pitch);
    uint32_t *sb = (uint32_t *)(xsum + 8 * (p.kr / p.gs));
    float *red = (float *)(sb + 16 * (p.kr / p.gs));

    const uint32_t *wbase = p.w + wb * p.w_batch_stride;
    const int64_t ra = min(n0 + r, p.N - 1), rb = min(n0 + r + 8, p.N - 1);
    const uint32_t *wa = wbase + ra * row_words + k0 * BITS / 32 + t * WPL;
    const uint32_t *wq = wbase + rb * row_words + k0 * BITS / 32 + t * WPL;

    // The warp's iterations.
    // The warp's iterations: whole groups, so every group is opened and closed by one warp.
    const int ipg = p.gs / IK;  // iterations per group (>= 1)
    const int it0 = (int)((int64_t)groups * warp / QMV_WARPS) * ipg;
    const int it1 = (int)((int64_t)groups * (warp + 1) / QMV_WARPS) * ipg;

    // Issue the first batch of weight loads before staging, so HBM latency overlaps it.
    uint32_t qa[QMV_UNROLL][WPL], qb[QMV_UNROLL][WPL];
#pragma unroll
    for (int u = 0; u < QMV_UNROLL; u++) {
        if (it0 + u < it1) {
            ldg_stream(qa[u], wa + (int64_t)(it0 + u) * 4 * WPL);
            ldg_stream(qb[u], wq + (int64_t)(it0 + u) * 4 * WPL);
        } else {
#pragma unroll
            for (int j = 0; j < WPL; j++) qa[u][j] = qb[u][j] = 0u;
        }
    }

    // ── stage activations (permuted), their group sums, and the scale/bias pairs ─────────
    {
        const __nv_bfloat16 *x = (const __nv_bfloat16 *)p.x + xb * p.x_batch_stride;
        const int blocks_per_row = kr / CODES;
        const int total = p.M * blocks_per_row;
        const int seg = p.gs / CODES;  // staging threads per group: a power of two <= 32
        for (int base = 0; base < total; base += QMV_WARPS * 32) {
            const int i = base + tid;
            const bool valid = i < total;
            int m = 0, blk = 0;
            float part = 0.f;
            if (valid) {
                m = i / blocks_per_row;
                blk = i - m * blocks_per_row;
                __nv_bfloat16 in[CODES], out[XREGS * 2];
                const __nv_bfloat16 *src = x + (int64_t)m * p.ldx + k0 + (int64_t)blk * CODES;
                if (p.x_vec) {
                    constexpr int VEC = CODES * 2 / 16 > 0 ? CODES * 2 / 16 : 1;
                    if (CODES * 2 >= 16) {
#pragma unroll
                        for (int v = 0; v < VEC; v++)
                            *reinterpret_cast<uint4 *>(in + 8 * v) = __ldg(reinterpret_cast<const uint4 *>(src) + v);
                    } else {
                        *reinterpret_cast<uint2 *>(in) = __ldg(reinterpret_cast<const uint2 *>(src));
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < CODES; j++) in[j] = src[j];
                }
#pragma unroll
                for (int j = 0; j < CODES; j++) part += __bfloat162float(in[j]);
                U::permute(in, out);
                uint32_t *dst = xs + (size_t)m * xs_pitch + (size_t)blk * XREGS;
#pragma unroll
                for (int j = 0; j < XREGS; j++)
                    dst[j] = (uint32_t)__bfloat16_as_ushort(out[2 * j]) | ((uint32_t)__bfloat16_as_ushort(out[2 * j + 1]) << 16);
            }
            // group sum over `seg` neighbouring lanes (segments never straddle a warp)
            for (int o = 1; o < seg; o <<= 1) part += __shfl_xor_sync(0xFFFFFFFFu, part, o);
            if (valid && (lane & (seg - 1)) == 0) xsum[m * groups + blk / seg] = part;
        }
        for (int i = p.M * groups + tid; i < 8 * groups; i += QMV_WARPS * 32) xsum[i] = 0.f;
        const __nv_bfloat16 *sc = (const __nv_bfloat16 *)p.scales + wb * p.s_batch_stride;
        const __nv_bfloat16 *bi = (const __nv_bfloat16 *)p.biases + wb * p.s_batch_stride;
        for (int i = tid; i < 16 * groups; i += QMV_WARPS * 32) {
            int rr = i / groups, g = i - rr * groups;
            int64_t row = min(n0 + rr, p.N - 1);
            size_t at = (size_t)(row * row_groups + g0 + g);
            sb[rr * groups + g] = (uint32_t)__bfloat16_as_ushort(sc[at]) | ((uint32_t)__bfloat16_as_ushort(bi[at]) << 16);
        }
    }
    __syncthreads();

    // ── main loop ───────────────────────────────────────────────────────────────────────
    float y[4] = {0.f, 0.f, 0.f, 0.f};    // rows r / r+8, activation rows 2t / 2t+1
    float acc[4] = {0.f, 0.f, 0.f, 0.f};  // the open group's sums
    const bool xrow = r < p.M;
    const uint32_t *xl = xs + (size_t)(xrow ? r : 0) * xs_pitch;

    for (int base = it0; base < it1; base += QMV_UNROLL) {
#pragma unroll
        for (int u = 0; u < QMV_UNROLL; u++) {
            const int it = base + u;
            if (it < it1) {
#pragma unroll
                for (int j = 0; j < WPL; j++) {
                    uint32_t ra_[REGS], rb_[REGS];
                    U::run(qa[u][j], ra_);
                    U::run(qb[u][j], rb_);
                    // activation registers of this word (zero for rows the product lacks)
                    uint32_t xr[XREGS];
                    const uint32_t *xp = xl + (size_t)((it * 4 + t) * WPL + j) * XREGS;
                    if (xrow) {
#pragma unroll
                        for (int v = 0; v < XREGS; v += 4) {
                            uint4 q = *reinterpret_cast<const uint4 *>(xp + v);
                            xr[v] = q.x; xr[v + 1] = q.y; xr[v + 2] = q.z; xr[v + 3] = q.w;
                        }
                    } else {
#pragma unroll
                        for (int v = 0; v < XREGS; v++) xr[v] = 0u;
                    }
#pragma unroll
                    for (int h = 0; h < REGS / 2; h++) {
                        uint32_t a[4] = {ra_[2 * h], rb_[2 * h], ra_[2 * h + 1], rb_[2 * h + 1]};
                        mma_bf16_16816(acc, a, xr[2 * h], xr[2 * h + 1]);
                    }
                }
                if ((it + 1) % ipg == 0) {
                    // close the group: y += s * acc + (b - OFFSET * s) * xsum
                    const int g = it / ipg;
                    uint32_t sa = sb[r * groups + g], sq = sb[(r + 8) * groups + g];
                    float s0 = __uint_as_float(sa << 16), b0 = __uint_as_float(sa & 0xFFFF0000u);
                    float s1 = __uint_as_float(sq << 16), b1 = __uint_as_float(sq & 0xFFFF0000u);
                    float x0 = xsum[(2 * t) * groups + g], x1 = xsum[(2 * t + 1) * groups + g];
                    float c0 = __fmaf_rn(-U::OFFSET, s0, b0), c1 = __fmaf_rn(-U::OFFSET, s1, b1);
                    y[0] += s0 * acc[0] + c0 * x0;
                    y[1] += s0 * acc[1] + c0 * x1;
                    y[2] += s1 * acc[2] + c1 * x0;
                    y[3] += s1 * acc[3] + c1 * x1;
                    acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
                }
            }
        }
        // next batch of loads
#pragma unroll
        for (int u = 0; u < QMV_UNROLL; u++) {
            const int it = base + QMV_UNROLL + u;
            if (it < it1) {
                ldg_stream(qa[u], wa + (int64_t)it * 4 * WPL);
                ldg_stream(qb[u], wq + (int64_t)it * 4 * WPL);
            }
        }
    }

    // ── reduce the warps' partial sums ──────────────────────────────────────────────────
    red[warp * 128 + r * 8 + 2 * t] = y[0];
    red[warp * 128 + r * 8 + 2 * t + 1] = y[1];
    red[warp * 128 + (r + 8) * 8 + 2 * t] = y[2];
    red[warp * 128 + (r + 8) * 8 + 2 * t + 1] = y[3];
    __syncthreads();
    const bool owner = tid < 128;  // thread (row, col) of the 16 x 8 output tile
    const int row = (tid >> 3) & 15, col = tid & 7;
    float total = 0.f;
    if (owner) {
#pragma unroll
        for (int w = 0; w < QMV_WARPS; w++) total += red[w * 128 + tid];
    }
    __nv_bfloat16 *out = (__nv_bfloat16 *)p.y + b * p.M * p.N;
    const bool store = owner && col < p.M && n0 + row < p.N;
    if (p.ksplit == 1) {
        if (store) out[(int64_t)col * p.N + n0 + row] = __float2bfloat16_rn(total);
        return;
    }
    // Split K: every block leaves its 16 x 8 partial in scratch; the block that arrives last
    // adds them in split order (so the result does not depend on arrival order) and rearms
    // the counter for the next launch.
    const int64_t tile = b * gridDim.x + blockIdx.x;
    float *part = p.partials + (tile * p.ksplit) * 128;
    if (owner) {
        __stcg(part + (int64_t)ks * 128 + tid, total);
        __threadfence();
    }
    __shared__ uint32_t arrived;
    __syncthreads();
    if (tid == 0) arrived = atomicAdd(p.counters + tile, 1u);
    __syncthreads();
    if (arrived != (uint32_t)p.ksplit - 1) return;
    __threadfence();
    if (owner) {
        float sum = 0.f;
        for (int s = 0; s < p.ksplit; s++) sum += __ldcg(part + (int64_t)s * 128 + tid);
        if (store) out[(int64_t)col * p.N + n0 + row] = __float2bfloat16_rn(sum);
    }
    if (tid == 0) p.counters[tile] = 0u;
}

// ── host side ──────────────────────────────────────────────────────────────────────────

static int wpl_for(int bits, int gs) {
    // words per lane per iteration, so that one quad (4 lanes) covers IK = 4*WPL*codes k-values
    // with IK dividing the group size
    switch (bits) {
    case 4: return gs == 32 ? 1 : gs == 64 ? 2 : 4;
    case 8: return gs == 32 ? 2 : 4;
    case 2: return gs == 64 ? 1 : gs == 128 ? 2 : 0;
    default: return 0;
    }
}

bool qmv_affine_eligible(int32_t mode, int32_t gs, int32_t bits, int32_t dtype, int32_t transpose, int64_t M,
                         int64_t N, int64_t K, const void *x, int64_t ldx, int64_t x_batch_stride, const uint32_t *w,
                         int64_t w_batch_stride) {
    (void)x; (void)ldx; (void)x_batch_stride;
    if (mode != NVC_AFFINE || dtype != NVC_BF16 || !transpose) return false;
    if (M < 1 || M > 8 || N < 1 || K < gs) return false;
    int wpl = wpl_for(bits, gs);
    if (wpl == 0) return false;
    int64_t row_words = K * bits / 32;
    if (row_words % wpl != 0 || w_batch_stride % wpl != 0 || ((uintptr_t)w % (4 * wpl)) != 0) return false;
    return true;
}

template <int BITS, int WPL>
static int32_t launch_qmv_cfg(nvc_device *dev, QmvParams &p, int64_t batch, size_t smem) {
    auto kernel = qmv_affine_kernel<BITS, WPL>;
    if (smem > 48 * 1024) NVC_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((unsigned)((p.N + 15) / 16), (unsigned)p.ksplit, (unsigned)batch);
    kernel<<<grid, QMV_WARPS * 32, smem, dev->stream>>>(p);
    return check_launch(dev, "qmv_affine_kernel");
}

int32_t launch_qmv_affine(nvc_device *dev, int32_t bits, QmvParams p, int64_t batch) {
    if (batch == 0 || p.N == 0 || p.M == 0) return NVC_OK;
    if (batch > 65535) return set_error(NVC_ERR_UNSUPPORTED, "qmv: %lld batches exceed the grid limit", (long long)batch);
    const int wpl = wpl_for(bits, p.gs);
    const int codes = bits == 4 ? 8 : bits == 8 ? 4 : 16, xregs = bits == 2 ? 8 : 4;
    const int64_t groups = p.K / p.gs;
    const int64_t tiles = (p.N + 15) / 16 * batch;
    auto smem_for = [&](int64_t kr) {
        return (size_t)(p.M * (kr / codes * xregs + 4) + 24 * (kr / p.gs) + QMV_WARPS * 128) * 4;
    };
    // Split K until the grid covers the machine about twice, keeping at least one group per
    // warp and the staged activations within 64 KiB.
    int64_t want = (2 * (int64_t)dev->prop.multiProcessorCount + tiles - 1) / tiles;
    int64_t max_split = groups / QMV_WARPS > 0 ? groups / QMV_WARPS : 1;
    int64_t ksplit = want < 1 ? 1 : want > max_split ? max_split : want;
    if (const char *e = getenv("NUVEC_QMV_KSPLIT")) {
        int64_t v = atoll(e);
        if (v >= 1) ksplit = v > groups ? groups : v;
    }
    int64_t kr = (groups + ksplit - 1) / ksplit * p.gs;
    while (smem_for(kr) > 64 * 1024 && kr > p.gs) {
        ksplit++;
        kr = (groups + ksplit - 1) / ksplit * p.gs;
    }
    ksplit = (p.K + kr - 1) / kr;
    p.kr = (int32_t)kr;
    p.ksplit = (int32_t)ksplit;
    p.partials = nullptr;
    p.counters = nullptr;
    if (ksplit > 1) {
        void *scratch = nullptr;
        NVC_TRY(ensure_scratch(dev, (size_t)tiles * ksplit * 128 * sizeof(float), &scratch));
        p.partials = (float *)scratch;
        NVC_TRY(ensure_counters(dev, (size_t)tiles, &p.counters));
    }
    const size_t smem = smem_for(kr);
#define NVC_QMV(B, W) if (bits == B && wpl == W) return launch_qmv_cfg<B, W>(dev, p, batch, smem);
    NVC_QMV(4, 1) NVC_QMV(4, 2) NVC_QMV(4, 4) NVC_QMV(8, 2) NVC_QMV(8, 4) NVC_QMV(2, 1) NVC_QMV(2, 2)
#undef NVC_QMV
    return set_error(NVC_ERR_UNSUPPORTED, "qmv: no kernel for %d bits, group size %d", bits, p.gs);
}

}  // namespace nvc
