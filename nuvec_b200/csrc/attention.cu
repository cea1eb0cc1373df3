// Decode attention over an affine-quantized KV cache: fast::quantized_attention
// (crates/nuvec-core/src/fast.rs:694-722, fast/imp.rs:3940-4096; mlx-lm's quantized KV cache),
//
//     out[b, h, 0, :] = softmax(scale * q[b, h, 0, :] . K[b, h / rep, s, :] over s [, sinks[h]]) . V[b, h / rep, s, :]
//
// for every query row of every head (no mask; a row at a time), K and V as codes uint32 [B, Hkv, S, D * bits / 32] with scales and
// biases [B, Hkv, S, D / group_size], rep = Hq / Hkv query heads per key head, and an optional
// per-head sink that joins the softmax's denominator only.  The shapes the reference's kernel takes
// (fast/imp.rs:3944-3993): D 64 or 128, 3, 4 or 8 bits, groups of 32, 64 or 128, rep 1, 2, 4 or 8.
// Like that kernel it dequantizes in registers and keeps everything in float32, so it is within
// the float bound of attention over the dequantized cache (the bound the reference's test sets,
// crates/nuvec-core/tests/quantized.rs:1964-2031), not the bits of mlx-lm's composition, which
// rounds the scores to the queries' type.
//
// A cache is a view of a longer allocation (capacity beyond the keys): `capacity` is the number
// of rows between consecutive heads of every cache tensor.
//
// Every form splits the keys: one block of four warps per (split, key head, batch) walks its keys in tiles of
// 128 with a running maximum and denominator per query head, and qattn_combine merges the splits (and the sink)
// and rounds to the output type.  qattn_split_kernel (float32, and 3-bit codes) works on the CUDA cores:
// scores by one thread per key, which reads the key's codes once and multiplies them with all rep query rows
// (float32 queries in shared memory, the group's scale and bias applied per group: s * sum(code * q) +
// b * sum(q)); values staged in shared memory with 16-byte loads, 64 threads x 2 key halves each own D / 64
// output columns and accumulate p * (s * code + b).  qattn_mma_kernel (16-bit types, 4- and 8-bit codes) does
// both products on the tensor cores; see there.
#include "common.cuh"

#include <mutex>

namespace nvc {

constexpr int QA_THREADS = 128, QA_TILE = 128, QA_MAX_REP = 8;
#ifndef QA_MMA_BLOCKS
#define QA_MMA_BLOCKS 3
#endif

struct QAttnParams {
    const void *q;                               // [B, Hq, L, D]
    const uint32_t *kw, *vw;                     // codes
    const void *ks, *kb, *vs, *vb;               // scales, biases
    const void *sinks;                           // [Hq] or null
    float *part;                                 // [B, Hq, splits, D + 2]: acc, m, l
    void *out;                                   // [B, Hq, L, D]
    int32_t B, Hq, Hkv, S, capacity, splits, chunk;
    int32_t L, l;                                // query rows per head, and the row this launch attends for
    float scale;
};

// Code d of a row of BITS-bit codes packed low bits first (kernels.rs:749-756); `row` may be registers
// (d known at compile time after unrolling) or shared memory.
template <int BITS>
__device__ __forceinline__ uint32_t qa_code(const uint32_t *row, int d) {
    if (BITS == 8) return (row[d >> 2] >> (8 * (d & 3))) & 0xFFu;
    if (BITS == 4) return (row[d >> 3] >> (4 * (d & 7))) & 0xFu;
    const int bit = d * 3, w = bit >> 5, off = bit & 31;
    uint32_t v = row[w] >> off;
    if (off > 29) v |= row[w + 1] << (32 - off);
    return v & 7u;
}

// an integer below 2^23 as a float without the conversion unit (a quarter-rate instruction otherwise)
__device__ __forceinline__ float qa_float(uint32_t c) { return __uint_as_float(0x4B000000u | c) - 8388608.0f; }

template <typename T, int BITS, int D, int GS>
__global__ void __launch_bounds__(QA_THREADS, 5) qattn_split_kernel(QAttnParams p) {
    constexpr int W = D * BITS / 32, G = D / GS, DPT = D / 64;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the combine kernel's blocks may become resident meanwhile
    const int split = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
    const int rep = p.Hq / p.Hkv, t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const int s0 = split * p.chunk, s1 = min(p.S, s0 + p.chunk);

    __shared__ __align__(16) float qs[D][QA_MAX_REP];          // scaled queries, [d][head]
    __shared__ float qsum[G][QA_MAX_REP];                      // their sums per group
    __shared__ __align__(16) float pr[QA_TILE][QA_MAX_REP];    // the tile's probabilities, [key][head]
    __shared__ float wred[2][4][QA_MAX_REP];                   // per-warp maxima / sums
    __shared__ __align__(16) uint32_t vrow[QA_TILE][W];        // the tile's value codes
    __shared__ float2 vsb[QA_TILE][G];                         // their (scale, bias)
    __shared__ float accx[64][DPT][QA_MAX_REP];                // second key half's sums, for the merge

    for (int i = t; i < D * QA_MAX_REP; i += QA_THREADS) {
        const int d = i / QA_MAX_REP, h = i % QA_MAX_REP;
        qs[d][h] = h < rep ? __fmul_rn(DT<T>::load((const T *)p.q, (((size_t)b * p.Hq + hk * rep + h) * p.L + p.l) * D + d), p.scale) : 0.0f;
    }
    __syncthreads();
    if (t < G * QA_MAX_REP) {
        const int g = t / QA_MAX_REP, h = t % QA_MAX_REP;
        float s = 0.0f;
        for (int d = 0; d < GS; d++) s += qs[g * GS + d][h];
        qsum[g][h] = s;
    }
    __syncthreads();

    const size_t head_row = ((size_t)b * p.Hkv + hk) * p.capacity;
    float m[QA_MAX_REP], l[QA_MAX_REP], acc[DPT][QA_MAX_REP];
#pragma unroll
    for (int h = 0; h < QA_MAX_REP; h++) {
        m[h] = -INFINITY;
        l[h] = 0.0f;
#pragma unroll
        for (int j = 0; j < DPT; j++) acc[j][h] = 0.0f;
    }
    const int dl = t & 63, half = t >> 6;  // value phase: columns dl * DPT .. , keys half * 64 ..

    for (int base = s0; base < s1; base += QA_TILE) {
        // ── scores of key base + t ──
        const int key = base + t;
        const bool valid = key < s1;
        float dot[QA_MAX_REP];
#pragma unroll
        for (int h = 0; h < QA_MAX_REP; h++) dot[h] = 0.0f;
        if (valid) {
            uint32_t row[W];
            const uint32_t *src = p.kw + (head_row + key) * W;
            if (W % 4 == 0) {
#pragma unroll
                for (int i = 0; i < W / 4; i++) {
                    const uint4 v = reinterpret_cast<const uint4 *>(src)[i];
                    row[4 * i] = v.x; row[4 * i + 1] = v.y; row[4 * i + 2] = v.z; row[4 * i + 3] = v.w;
                }
            } else {
#pragma unroll
                for (int i = 0; i < W / 2; i++) {
                    const uint2 v = reinterpret_cast<const uint2 *>(src)[i];
                    row[2 * i] = v.x; row[2 * i + 1] = v.y;
                }
            }
#pragma unroll
            for (int g = 0; g < G; g++) {
                float a[QA_MAX_REP];
#pragma unroll
                for (int h = 0; h < QA_MAX_REP; h++) a[h] = 0.0f;
#pragma unroll
                for (int d = g * GS; d < (g + 1) * GS; d++) {
                    const float c = qa_float(qa_code<BITS>(row, d));
                    const float4 q0 = *reinterpret_cast<const float4 *>(&qs[d][0]);
                    a[0] = fmaf(c, q0.x, a[0]); a[1] = fmaf(c, q0.y, a[1]); a[2] = fmaf(c, q0.z, a[2]); a[3] = fmaf(c, q0.w, a[3]);
                    if (rep > 4) {
                        const float4 q1 = *reinterpret_cast<const float4 *>(&qs[d][4]);
                        a[4] = fmaf(c, q1.x, a[4]); a[5] = fmaf(c, q1.y, a[5]); a[6] = fmaf(c, q1.z, a[6]); a[7] = fmaf(c, q1.w, a[7]);
                    }
                }
                const float sg = DT<T>::load((const T *)p.ks, (head_row + key) * G + g), bg = DT<T>::load((const T *)p.kb, (head_row + key) * G + g);
#pragma unroll
                for (int h = 0; h < QA_MAX_REP; h++) dot[h] = fmaf(sg, a[h], fmaf(bg, qsum[g][h], dot[h]));
            }
        }
        // ── the tile's values into shared memory (all threads) ──
        {
            const int keys = min(QA_TILE, s1 - base);
            constexpr int U = W % 4 == 0 ? 4 : 2;  // words per load
            const uint32_t *src = p.vw + (head_row + base) * W;
            for (int i = t; i < keys * W / U; i += QA_THREADS) {
                if (U == 4) reinterpret_cast<uint4 *>(&vrow[0][0])[i] = reinterpret_cast<const uint4 *>(src)[i];
                else reinterpret_cast<uint2 *>(&vrow[0][0])[i] = reinterpret_cast<const uint2 *>(src)[i];
            }
            for (int i = t; i < keys * G; i += QA_THREADS)
                vsb[0][i] = make_float2(DT<T>::load((const T *)p.vs, (head_row + base) * G + i), DT<T>::load((const T *)p.vb, (head_row + base) * G + i));
        }
        // ── running maximum and denominator per head ──
        float corr[QA_MAX_REP];
#pragma unroll
        for (int h = 0; h < QA_MAX_REP; h++) {
            float v = valid ? dot[h] : -INFINITY;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
            if (lane == 0) wred[0][warp][h] = v;
        }
        __syncthreads();
#pragma unroll
        for (int h = 0; h < QA_MAX_REP; h++) {
            const float mn = fmaxf(fmaxf(m[h], fmaxf(wred[0][0][h], wred[0][1][h])), fmaxf(wred[0][2][h], wred[0][3][h]));
            corr[h] = m[h] == -INFINITY ? 0.0f : expf(m[h] - mn);
            m[h] = mn;
            const float e = valid ? expf(dot[h] - mn) : 0.0f;
            pr[t][h] = e;
            float v = e;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
            if (lane == 0) wred[1][warp][h] = v;
        }
        __syncthreads();
#pragma unroll
        for (int h = 0; h < QA_MAX_REP; h++) l[h] = fmaf(l[h], corr[h], (wred[1][0][h] + wred[1][1][h]) + (wred[1][2][h] + wred[1][3][h]));
        // ── values: columns dl * DPT .. of keys half * 64 .. + 63 of the tile ──
#pragma unroll
        for (int j = 0; j < DPT; j++)
#pragma unroll
            for (int h = 0; h < QA_MAX_REP; h++) acc[j][h] *= corr[h];
        const int kend = min(64, s1 - base - half * 64);
        for (int kk = 0; kk < kend; kk++) {
            const int s = half * 64 + kk;
            const float4 p0 = *reinterpret_cast<const float4 *>(&pr[s][0]);
            float4 p1 = make_float4(0.f, 0.f, 0.f, 0.f);
            if (rep > 4) p1 = *reinterpret_cast<const float4 *>(&pr[s][4]);
#pragma unroll
            for (int j = 0; j < DPT; j++) {
                const int d = dl * DPT + j;
                const float2 sb = vsb[s][d / GS];
                const float v = fmaf(sb.x, qa_float(qa_code<BITS>(vrow[s], d)), sb.y);
                acc[j][0] = fmaf(p0.x, v, acc[j][0]); acc[j][1] = fmaf(p0.y, v, acc[j][1]);
                acc[j][2] = fmaf(p0.z, v, acc[j][2]); acc[j][3] = fmaf(p0.w, v, acc[j][3]);
                if (rep > 4) {
                    acc[j][4] = fmaf(p1.x, v, acc[j][4]); acc[j][5] = fmaf(p1.y, v, acc[j][5]);
                    acc[j][6] = fmaf(p1.z, v, acc[j][6]); acc[j][7] = fmaf(p1.w, v, acc[j][7]);
                }
            }
        }
        __syncthreads();  // pr, vrow, vsb and wred are rewritten by the next tile
    }

    // ── the two key halves together, then this split's partial result ──
    if (half == 1) {
#pragma unroll
        for (int j = 0; j < DPT; j++)
#pragma unroll
            for (int h = 0; h < QA_MAX_REP; h++) accx[dl][j][h] = acc[j][h];
    }
    __syncthreads();
    if (half == 0) {
#pragma unroll
        for (int h = 0; h < QA_MAX_REP; h++) {
            if (h >= rep) break;
            float *dst = p.part + (((size_t)b * p.Hq + hk * rep + h) * p.splits + split) * (D + 2);
#pragma unroll
            for (int j = 0; j < DPT; j++) dst[dl * DPT + j] = acc[j][h] + accx[dl][j][h];
            if (dl == 0) {
                dst[D] = m[h];
                dst[D + 1] = l[h];
            }
        }
    }
}

// ── the tensor-core form (16-bit types, 4- and 8-bit codes) ─────────────────────────────────────────────
// mma.sync m16n8k16 (float16 operands, float32 accumulators): the rows of the A operand are the key head's
// query heads (8 of the 16 rows at most are used), a code enters as the exact float16 integer 1024 + code
// (0x6400 | code), and the offset is taken out again with sums the kernel keeps anyway:
//   scores   S_g[h, key] = sum over the group's dims of q[h, d] * (1024 + code[key, d])        (tensor cores)
//            score[h, key] = sum_g  s_g[key] * (S_g - 1024 * qsum_g[h]) + b_g[key] * qsum_g[h]
//   values   O[h, d] += sum over keys of (p[h, key] * s_g(d)[key]) * (1024 + code[key, d])      (tensor cores)
//            out[h, d] = O[h, d] + sum over keys of (p * b_g(d)[key] - 1024 * p * s_g(d)[key])
// A warp owns 32 keys of a tile of 128: its score accumulators (C fragments, 16 heads x 8 keys) are, pairwise,
// exactly the A fragments (16 heads x 16 keys) of its value products, so the probabilities never leave
// registers; the four warps' outputs are added at the end.  A tile's codes travel into shared memory with cp.async a
// tile ahead (two sets of buffers), its scales and biases through registers.  q * scale and p * s are rounded to float16
// (11 significant bits, three more than the bfloat16 the reference's composition rounds them to).
__device__ __forceinline__ void qa_mma(float (&c)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    const uint32_t zero = 0u;  // rows 8-15 of A (no heads there)
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(zero), "r"(a2), "r"(zero), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t qa_pack_f16(float lo, float hi) {
    const __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&v);
}
__device__ __forceinline__ float2 qa_unpack_f16(uint32_t v) { return __half22float2(*reinterpret_cast<const __half2 *>(&v)); }

__device__ __forceinline__ void qa_cp16(void *dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ size_t head_row_of(const QAttnParams &p, int b, int hk) { return ((size_t)b * p.Hkv + hk) * p.capacity; }

template <typename T, int BITS, int D, int GS>
__global__ void __launch_bounds__(QA_THREADS, QA_MMA_BLOCKS) qattn_mma_kernel(QAttnParams p) {
    static_assert(BITS == 4 || BITS == 8, "codes that fill bytes");
    constexpr int W = D * BITS / 32, G = D / GS, KS = D / 16, NBD = D / 8, WP = W + 4;  // WP: padded row of the value tile
    constexpr int KS_PER_G = GS / 16, NBD_PER_G = GS / 8;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the combine kernel's blocks may become resident meanwhile
    const int split = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
    const int rep = p.Hq / p.Hkv, t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const int g8 = lane >> 2, c = lane & 3;  // the fragments' group (a head, a key or a dim) and pair index
    const int s0 = split * p.chunk, s1 = min(p.S, s0 + p.chunk);
    const bool head = g8 < rep;

    // Two sets of tile buffers: the next tile's codes arrive (cp.async) while the current tile multiplies.  Rows are
    // padded by four words: the eight rows (keys) or four rows (values) a fragment reads at once fall into distinct banks.
    __shared__ float wred[2][4][8];
    constexpr int KP = W + 4;
    constexpr int TILE_WORDS = QA_TILE * KP, RWORDS = 4 * 8 * D;
    extern __shared__ __align__(16) uint32_t qa_dyn[];
    uint32_t *kbuf = qa_dyn;                        // [2][QA_TILE * KP]
    uint32_t *vbuf = kbuf + 2 * TILE_WORDS;         // [2][QA_TILE * WP]; after the last tile the warps' sums [4][8][D]
    float4 *sbuf = reinterpret_cast<float4 *>(vbuf + (2 * TILE_WORDS > RWORDS ? 2 * TILE_WORDS : RWORDS));  // [2][QA_TILE][G]
    auto fetch_codes = [&](int base, int buf) {
        const int keys = min(QA_TILE, s1 - base);
        const uint32_t *ksrc = p.kw + (head_row_of(p, b, hk) + base) * W, *vsrc = p.vw + (head_row_of(p, b, hk) + base) * W;
        for (int i = t; i < keys * W / 4; i += QA_THREADS) {
            const int row = (4 * i) / W, col = (4 * i) % W;
            qa_cp16(kbuf + buf * TILE_WORDS + row * KP + col, ksrc + 4 * i);
            qa_cp16(vbuf + buf * TILE_WORDS + row * WP + col, vsrc + 4 * i);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    auto fetch_scales = [&](int base, float4 (&r)[G]) {  // thread t: key t of the tile
        const int keys = min(QA_TILE, s1 - base);
#pragma unroll
        for (int g = 0; g < G; g++) {
            const size_t at = (head_row_of(p, b, hk) + base + min(t, keys - 1)) * G + g;
            r[g] = make_float4(DT<T>::load((const T *)p.ks, at), DT<T>::load((const T *)p.kb, at), DT<T>::load((const T *)p.vs, at),
                               DT<T>::load((const T *)p.vb, at));
        }
    };

    // the head's scaled queries as A fragments, and their sums per group (of the rounded values)
    uint32_t qa0[KS], qa2[KS];
    float qsum[G];
#pragma unroll
    for (int g = 0; g < G; g++) qsum[g] = 0.0f;
    {
        const T *q = (const T *)p.q + (((size_t)b * p.Hq + hk * rep + (head ? g8 : 0)) * p.L + p.l) * D;
#pragma unroll
        for (int ks = 0; ks < KS; ks++) {
            const int d = 16 * ks + 2 * c;
            qa0[ks] = head ? qa_pack_f16(DT<T>::load(q, d) * p.scale, DT<T>::load(q, d + 1) * p.scale) : 0u;
            qa2[ks] = head ? qa_pack_f16(DT<T>::load(q, d + 8) * p.scale, DT<T>::load(q, d + 9) * p.scale) : 0u;
            const float2 u = qa_unpack_f16(qa0[ks]), v = qa_unpack_f16(qa2[ks]);
            qsum[ks / KS_PER_G] += (u.x + u.y) + (v.x + v.y);
        }
#pragma unroll
        for (int g = 0; g < G; g++) {
            qsum[g] += __shfl_xor_sync(0xFFFFFFFFu, qsum[g], 1);
            qsum[g] += __shfl_xor_sync(0xFFFFFFFFu, qsum[g], 2);
        }
    }

    float m = -INFINITY, l = 0.0f;  // of head g8
    float oc[NBD][4], side[G];      // outputs [head g8][dims 8 nbd + 2 c, + 1] (rows 8-15 idle); bias / offset terms per group
#pragma unroll
    for (int i = 0; i < NBD; i++) oc[i][0] = oc[i][1] = oc[i][2] = oc[i][3] = 0.0f;
#pragma unroll
    for (int g = 0; g < G; g++) side[g] = 0.0f;

    float4 nsb[G];
    if (s0 < s1) {
        fetch_codes(s0, 0);
        fetch_scales(s0, nsb);
#pragma unroll
        for (int g = 0; g < G; g++) sbuf[t * G + g] = nsb[g];
    }
    int buf = 0;
    for (int base = s0; base < s1; base += QA_TILE, buf ^= 1) {
        const int keys = min(QA_TILE, s1 - base);
        const bool more = base + QA_TILE < s1;
        // the next tile's codes start travelling into the other buffers, its scales into registers
        if (more) {
            fetch_codes(base + QA_TILE, buf ^ 1);
            fetch_scales(base + QA_TILE, nsb);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const uint32_t *ktile = kbuf + buf * TILE_WORDS, *vtile = vbuf + buf * TILE_WORDS;
        const float4(*sbt)[G] = reinterpret_cast<const float4(*)[G]>(sbuf + buf * QA_TILE * G);
        // ── scores of the warp's 32 keys: four blocks of 8 keys ──
        float sc[4][2];
#pragma unroll
        for (int nb = 0; nb < 4; nb++) {
            const int kfrag = warp * 32 + nb * 8;                       // first key of the block, within the tile
            const int krow = min(kfrag + g8, keys - 1);                 // the key whose codes this lane feeds (clamped: masked below)
            const uint32_t *row = ktile + krow * KP;
            float cg[G][4];
#pragma unroll
            for (int g = 0; g < G; g++) cg[g][0] = cg[g][1] = cg[g][2] = cg[g][3] = 0.0f;
#pragma unroll
            for (int q4 = 0; q4 < W / 4; q4++) {
                const uint4 v = reinterpret_cast<const uint4 *>(row)[q4];
                const uint32_t w[4] = {v.x, v.y, v.z, v.w};
                if (BITS == 4) {
                    // words 4 q4 .. + 3 = dims 32 q4 .. + 31 = two steps of 16 dims; the lane's codes are byte c of every word
#pragma unroll
                    for (int half = 0; half < 2; half++) {
                        const int ks = 2 * q4 + half;
                        uint32_t bf[2];
#pragma unroll
                        for (int j = 0; j < 2; j++) {
                            const uint32_t byte = __byte_perm(w[2 * half + j], 0, 0x4440 | c);
                            bf[j] = ((byte | (byte << 12)) & 0x000F000Fu) | 0x64006400u;
                        }
                        qa_mma(cg[ks / KS_PER_G], qa0[ks], qa2[ks], bf[0], bf[1]);
                    }
                } else {
                    // words 4 q4 .. + 3 = dims 16 q4 .. + 15 = one step; dims 2 c, 2 c + 1 are a half of word c / 2, dims + 8 of word 2 + c / 2
                    const int ks = q4;
                    const uint32_t lo = (c & 2) ? w[1] : w[0], hi = (c & 2) ? w[3] : w[2];
                    const uint32_t sel = (c & 1) ? 0x4342u : 0x4140u;
                    qa_mma(cg[ks / KS_PER_G], qa0[ks], qa2[ks], __byte_perm(lo, 0, sel) | 0x64006400u, __byte_perm(hi, 0, sel) | 0x64006400u);
                }
            }
            // the C fragment holds [head g8][keys kfrag + 2 c, + 1]
#pragma unroll
            for (int j = 0; j < 2; j++) {
                const int key = min(kfrag + 2 * c + j, keys - 1);
                float sv = 0.0f;
#pragma unroll
                for (int g = 0; g < G; g++) {
                    const float4 sb = sbt[key][g];
                    sv = fmaf(sb.x, cg[g][j] - 1024.0f * qsum[g], fmaf(sb.y, qsum[g], sv));
                }
                sc[nb][j] = sv;
            }
        }
        // ── running maximum and denominator of head g8 ──
        float tmax = -INFINITY;
#pragma unroll
        for (int nb = 0; nb < 4; nb++)
#pragma unroll
            for (int j = 0; j < 2; j++) {
                const bool valid = head && warp * 32 + nb * 8 + 2 * c + j < keys;
                if (!valid) sc[nb][j] = -INFINITY;
                tmax = fmaxf(tmax, sc[nb][j]);
            }
        tmax = fmaxf(tmax, __shfl_xor_sync(0xFFFFFFFFu, tmax, 1));
        tmax = fmaxf(tmax, __shfl_xor_sync(0xFFFFFFFFu, tmax, 2));
        if (c == 0) wred[0][warp][g8] = tmax;
        __syncthreads();
        const float mn = fmaxf(fmaxf(m, fmaxf(wred[0][0][g8], wred[0][1][g8])), fmaxf(wred[0][2][g8], wred[0][3][g8]));
        const float corr = m == -INFINITY ? 0.0f : expf(m - mn);
        m = mn;
        float psum = 0.0f;
#pragma unroll
        for (int nb = 0; nb < 4; nb++)
#pragma unroll
            for (int j = 0; j < 2; j++) {
                sc[nb][j] = sc[nb][j] == -INFINITY ? 0.0f : expf(sc[nb][j] - mn);
                psum += sc[nb][j];
            }
        psum += __shfl_xor_sync(0xFFFFFFFFu, psum, 1);
        psum += __shfl_xor_sync(0xFFFFFFFFu, psum, 2);
        if (c == 0) wred[1][warp][g8] = psum;
        __syncthreads();
        l = fmaf(l, corr, (wred[1][0][g8] + wred[1][1][g8]) + (wred[1][2][g8] + wred[1][3][g8]));
#pragma unroll
        for (int i = 0; i < NBD; i++) {
            oc[i][0] *= corr;
            oc[i][1] *= corr;
        }
#pragma unroll
        for (int g = 0; g < G; g++) side[g] *= corr;
        // ── values: two steps of 16 keys; the probabilities times the keys' value scales are the A fragments ──
#pragma unroll
        for (int kk = 0; kk < 2; kk++) {
            const int r0 = warp * 32 + kk * 16 + 2 * c;  // the lane's keys within the tile: r0, r0 + 1, r0 + 8, r0 + 9
            uint32_t pa0[G], pa2[G];
#pragma unroll
            for (int g = 0; g < G; g++) {
                float ps[4], pb = 0.0f;
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int key = min(r0 + (i & 1) + 8 * (i >> 1), keys - 1);
                    const float pv = sc[2 * kk + (i >> 1)][i & 1];  // (zero for keys past the end)
                    const float4 sb = sbt[key][g];
                    ps[i] = pv * sb.z;
                    pb = fmaf(pv, sb.w, pb);
                }
                pa0[g] = qa_pack_f16(ps[0], ps[1]);
                pa2[g] = qa_pack_f16(ps[2], ps[3]);
                const float2 u = qa_unpack_f16(pa0[g]), v = qa_unpack_f16(pa2[g]);
                side[g] += pb - 1024.0f * ((u.x + u.y) + (v.x + v.y));
            }
            const uint32_t *v0 = vtile + r0 * WP, *v1 = v0 + WP, *v2 = v0 + 8 * WP, *v3 = v0 + 9 * WP;
#pragma unroll
            for (int nbd = 0; nbd < NBD; nbd++) {
                uint32_t b0, b1;
                if (BITS == 4) {
                    const int sh = 4 * g8;  // dim 8 nbd + g8 = nibble g8 of word nbd
                    b0 = (((v0[nbd] >> sh) & 0xFu) | (((v1[nbd] >> sh) & 0xFu) << 16)) | 0x64006400u;
                    b1 = (((v2[nbd] >> sh) & 0xFu) | (((v3[nbd] >> sh) & 0xFu) << 16)) | 0x64006400u;
                } else {
                    const int wd = 2 * nbd + (g8 >> 2), sh = 8 * (g8 & 3);  // byte g8 % 4 of word 2 nbd + g8 / 4
                    b0 = (((v0[wd] >> sh) & 0xFFu) | (((v1[wd] >> sh) & 0xFFu) << 16)) | 0x64006400u;
                    b1 = (((v2[wd] >> sh) & 0xFFu) | (((v3[wd] >> sh) & 0xFFu) << 16)) | 0x64006400u;
                }
                qa_mma(oc[nbd], pa0[nbd / NBD_PER_G], pa2[nbd / NBD_PER_G], b0, b1);
            }
        }
        if (more) {
#pragma unroll
            for (int g = 0; g < G; g++) sbuf[((buf ^ 1) * QA_TILE + t) * G + g] = nsb[g];
        }
        __syncthreads();  // this tile's buffers are refilled from the next iteration on; wred is rewritten by the next tile
    }

    // ── the four warps' outputs together, then this split's partial result ──
#pragma unroll
    for (int g = 0; g < G; g++) {
        side[g] += __shfl_xor_sync(0xFFFFFFFFu, side[g], 1);
        side[g] += __shfl_xor_sync(0xFFFFFFFFu, side[g], 2);
    }
    float *wsum = reinterpret_cast<float *>(vbuf);  // [warp][head][D]
    if (head) {
#pragma unroll
        for (int nbd = 0; nbd < NBD; nbd++) {
            float *dst = wsum + ((warp * 8 + g8) * D) + 8 * nbd + 2 * c;
            dst[0] = oc[nbd][0] + side[nbd / NBD_PER_G];
            dst[1] = oc[nbd][1] + side[nbd / NBD_PER_G];
        }
    }
    __syncthreads();
    for (int i = t; i < D * rep; i += QA_THREADS) {
        const int h = i / D, d = i % D;
        float *dst = p.part + (((size_t)b * p.Hq + hk * rep + h) * p.splits + split) * (D + 2);
        dst[d] = (wsum[(0 * 8 + h) * D + d] + wsum[(1 * 8 + h) * D + d]) + (wsum[(2 * 8 + h) * D + d] + wsum[(3 * 8 + h) * D + d]);
    }
    if (warp == 0 && c == 0 && head) {
        float *dst = p.part + (((size_t)b * p.Hq + hk * rep + g8) * p.splits + split) * (D + 2);
        dst[D] = m;
        dst[D + 1] = l;
    }
}

template <typename T, int D>
__global__ void __launch_bounds__(D) qattn_combine_kernel(QAttnParams p) {
    const int h = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
    asm volatile("griddepcontrol.wait;" ::: "memory");  // the partial results are the split kernel's
    const float *part = p.part + ((size_t)b * p.Hq + h) * p.splits * (D + 2);
    float mx = -INFINITY;
    for (int j = 0; j < p.splits; j++) mx = fmaxf(mx, part[j * (D + 2) + D]);
    const bool sink = p.sinks != nullptr;
    const float sv = sink ? DT<T>::load((const T *)p.sinks, h) : 0.0f;
    if (sink) mx = fmaxf(mx, sv);
    float num = 0.0f, den = sink ? expf(sv - mx) : 0.0f;
    for (int j = 0; j < p.splits; j++) {
        const float mj = part[j * (D + 2) + D];
        if (mj == -INFINITY) continue;
        const float w = expf(mj - mx);
        num = fmaf(w, part[j * (D + 2) + d], num);
        den = fmaf(w, part[j * (D + 2) + D + 1], den);
    }
    DT<T>::store((T *)p.out, (((size_t)b * p.Hq + h) * p.L + p.l) * D + d, den > 0.0f ? __fdiv_rn(num, den) : 0.0f);
}

// The combine kernel, launched so that it may become resident while the split kernel runs (NUVEC_PDL=0: plain order).
template <typename T, int D>
static int32_t qattn_combine(nvc_device *dev, const QAttnParams &p) {
    static const bool pdl = [] { const char *e = getenv("NUVEC_PDL"); return !(e && *e == '0'); }();
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)p.Hq, (unsigned)p.B);
    cfg.blockDim = dim3(D);
    cfg.stream = dev->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    NVC_CUDA(cudaLaunchKernelEx(&cfg, qattn_combine_kernel<T, D>, p));
    return check_launch(dev, "qattn_combine_kernel");
}

// 16-bit types with 4- or 8-bit codes run on the tensor cores (switch: NUVEC_QATTN_MMA=0)
static bool qattn_uses_mma(int dtype, int bits) {
    static const bool mma_on = !(getenv("NUVEC_QATTN_MMA") && atoi(getenv("NUVEC_QATTN_MMA")) == 0);
    return mma_on && dtype != NVC_F32 && bits != 3;
}

template <typename T, int BITS, int D, int GS>
static void qattn_launch_mma(nvc_device *dev, const QAttnParams &p, dim3 grid) {
    if constexpr (sizeof(T) == 2 && (BITS == 4 || BITS == 8) && D % GS == 0) {
        constexpr int W = D * BITS / 32, TILE_WORDS = QA_TILE * (W + 4), RWORDS = 4 * 8 * D;
        constexpr size_t smem = (size_t)(2 * TILE_WORDS + (2 * TILE_WORDS > RWORDS ? 2 * TILE_WORDS : RWORDS)) * 4 + 2 * QA_TILE * (D / GS) * 16;
        auto kernel = qattn_mma_kernel<T, BITS, D, GS>;
        static bool configured[64] = {};
        static std::mutex mu;
        if (dev->ordinal >= 0 && dev->ordinal < 64) {
            std::lock_guard<std::mutex> g(mu);
            if (!configured[dev->ordinal]) {
                cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                configured[dev->ordinal] = true;
            }
        }
        kernel<<<grid, QA_THREADS, smem, dev->stream>>>(p);
    }
}

template <typename T, int BITS, int D>
static int32_t qattn_launch(nvc_device *dev, const QAttnParams &p, int gs) {
    dim3 grid((unsigned)p.splits, (unsigned)p.Hkv, (unsigned)p.B);
    if (qattn_uses_mma(sizeof(T) == 2 ? NVC_F16 : NVC_F32, BITS)) {
        if (gs == 32) qattn_launch_mma<T, BITS, D, 32>(dev, p, grid);
        else if (gs == 64) qattn_launch_mma<T, BITS, D, 64>(dev, p, grid);
        else qattn_launch_mma<T, BITS, D, D == 128 ? 128 : 64>(dev, p, grid);
        NVC_TRY(check_launch(dev, "qattn_mma_kernel"));
        return qattn_combine<T, D>(dev, p);
    }
    if (gs == 32) qattn_split_kernel<T, BITS, D, 32><<<grid, QA_THREADS, 0, dev->stream>>>(p);
    else if (gs == 64) qattn_split_kernel<T, BITS, D, 64><<<grid, QA_THREADS, 0, dev->stream>>>(p);
    else if (D == 128) qattn_split_kernel<T, BITS, D, D == 128 ? 128 : 64><<<grid, QA_THREADS, 0, dev->stream>>>(p);
    NVC_TRY(check_launch(dev, "qattn_split_kernel"));
    return qattn_combine<T, D>(dev, p);
}

template <typename T>
static int32_t qattn_typed(nvc_device *dev, const QAttnParams &p, int bits, int d, int gs) {
    if (d == 128) {
        if (bits == 3) return qattn_launch<T, 3, 128>(dev, p, gs);
        if (bits == 4) return qattn_launch<T, 4, 128>(dev, p, gs);
        return qattn_launch<T, 8, 128>(dev, p, gs);
    }
    if (bits == 3) return qattn_launch<T, 3, 64>(dev, p, gs);
    if (bits == 4) return qattn_launch<T, 4, 64>(dev, p, gs);
    return qattn_launch<T, 8, 64>(dev, p, gs);
}

}  // namespace nvc

using namespace nvc;

extern "C" int32_t nvc_quantized_attention(nvc_device *dev, const nvc_quant *quant, int32_t dtype, const void *q, const uint32_t *k_codes,
                                           const void *k_scales, const void *k_biases, const uint32_t *v_codes, const void *v_scales,
                                           const void *v_biases, const void *sinks, int64_t B, int64_t Hq, int64_t Hkv, int64_t L, int64_t S,
                                           int64_t D, int64_t capacity, float scale, int32_t causal, void *out) {
    NVC_TRY(make_current(dev));
    NVC_TRY(check_quant("quantized_attention", quant));
    if (quant->mode != NVC_AFFINE) return set_error(NVC_ERR_INVALID_ARGUMENT, "quantized_attention: keys and values need one affine quantization");
    const int bits = quant->bits, gs = quant->group_size;
    if (dtype != NVC_F16 && dtype != NVC_BF16 && dtype != NVC_F32) return set_error(NVC_ERR_UNSUPPORTED, "quantized_attention: unsupported dtype %d", dtype);
    if (B < 0 || Hq < 0 || Hkv < 0 || L < 0 || S < 0 || capacity < S) return set_error(NVC_ERR_INVALID_ARGUMENT, "quantized_attention: invalid shape");
    if (L > 64) return set_error(NVC_ERR_UNSUPPORTED, "quantized_attention: %lld query rows per head (the cache is read once per row: up to 64)", (long long)L);
    if ((D != 64 && D != 128) || (bits != 3 && bits != 4 && bits != 8) || D % gs != 0)
        return set_error(NVC_ERR_UNSUPPORTED, "quantized_attention: head size %lld with %d bits in groups of %d (64 or 128; 3, 4 or 8; a group within a head)",
                         (long long)D, bits, gs);
    if (B * Hq * L == 0) return NVC_OK;
    if (Hkv <= 0 || Hq % Hkv != 0) return set_error(NVC_ERR_INVALID_ARGUMENT, "quantized_attention: %lld query heads over %lld key heads", (long long)Hq, (long long)Hkv);
    const int64_t rep = Hq / Hkv;
    if (rep != 1 && rep != 2 && rep != 4 && rep != 8) return set_error(NVC_ERR_UNSUPPORTED, "quantized_attention: %lld query heads per key head (1, 2, 4 or 8)", (long long)rep);
    if (B > 65535 || Hkv > 65535 || S > INT32_MAX || capacity > INT32_MAX) return set_error(NVC_ERR_UNSUPPORTED, "quantized_attention: too long");
    if (!q || !out || (S > 0 && (!k_codes || !k_scales || !k_biases || !v_codes || !v_scales || !v_biases)))
        return set_error(NVC_ERR_INVALID_ARGUMENT, "quantized_attention: null operand");
    if (((uintptr_t)k_codes | (uintptr_t)v_codes) % 16 != 0) return set_error(NVC_ERR_UNSUPPORTED, "quantized_attention: the codes must be 16-byte aligned");

    // splits: one wave of as many blocks as stay resident together (what their registers allow: three of the
    // tensor-core kernel, five of the other, per multiprocessor), whole tiles of 128 keys each
    const int64_t tiles = S > 0 ? (S + QA_TILE - 1) / QA_TILE : 1;
    int per_sm = 5;
    if (qattn_uses_mma(dtype, bits)) {
        // (the tensor-core kernel's two sets of tile buffers decide how many blocks stay resident)
        const int64_t tile_words = QA_TILE * (D * bits / 32 + 4), sum_words = 4 * 8 * D;
        const int64_t smem = (2 * tile_words + (2 * tile_words > sum_words ? 2 * tile_words : sum_words)) * 4 + 2 * QA_TILE * (D / gs) * 16;
        per_sm = (int)((227 * 1024) / (smem + 1024 + 256));
        if (per_sm > QA_MMA_BLOCKS) per_sm = QA_MMA_BLOCKS;
        if (per_sm < 1) per_sm = 1;
    }
    int64_t splits = per_sm * (int64_t)dev->prop.multiProcessorCount / (B * Hkv);
    if (splits > tiles) splits = tiles;
    if (splits < 1) splits = 1;
    const int64_t chunk = (tiles + splits - 1) / splits * QA_TILE;
    splits = S > 0 ? (S + chunk - 1) / chunk : 1;
    // the splits' partial results: the handle's scratch block (reused between calls in stream order; it grows outside
    // recorded steps only)
    const size_t part_bytes = (size_t)B * Hq * splits * (D + 2) * sizeof(float);
    if (dev->capturing && dev->scratch_bytes < part_bytes)
        return set_error(NVC_ERR_UNSUPPORTED, "quantized_attention: %zu bytes of scratch inside a recorded step (run the shape once before recording)",
                         part_bytes);
    void *part = nullptr;
    NVC_TRY(ensure_scratch(dev, part_bytes, &part));
    QAttnParams p{q, k_codes, v_codes, k_scales, k_biases, v_scales, v_biases, sinks, (float *)part, out,
                  (int32_t)B, (int32_t)Hq, (int32_t)Hkv, (int32_t)S, (int32_t)capacity, (int32_t)splits, (int32_t)chunk, (int32_t)L, 0, scale};
    int32_t rc = NVC_OK;
    // every query row attends to all the keys (or, causal, to those up to its position); a row at a time (the partial
    // results are reused in stream order)
    // (causal: query row l is the position S - L + l and attends to the keys up to it)
    for (int64_t l = 0; l < L && rc == NVC_OK; l++) {
        p.l = (int32_t)l;
        if (causal) p.S = (int32_t)(S - (L - 1 - l) > 0 ? S - (L - 1 - l) : 0);
        rc = dtype == NVC_F16 ? qattn_typed<__half>(dev, p, bits, (int)D, gs)
             : dtype == NVC_BF16 ? qattn_typed<__nv_bfloat16>(dev, p, bits, (int)D, gs) : qattn_typed<float>(dev, p, bits, (int)D, gs);
    }
    return rc;
}
