// Decode attention over an affine-quantized KV cache: fast::quantized_attention
// (crates/nuvec-core/src/fast.rs:694-722, fast/imp.rs:3940-4096; mlx-lm's quantized KV cache),
//
//     out[b, h, 0, :] = softmax(scale * q[b, h, 0, :] . K[b, h / rep, s, :] over s [, sinks[h]]) . V[b, h / rep, s, :]
//
// for one query row per head, K and V as codes uint32 [B, Hkv, S, D * bits / 32] with scales and
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
// Two kernels.  qattn_split: one block per (split of the keys, key head, batch) walks its keys in
// tiles of 128 with a running maximum and denominator per query head.  Scores: one thread per key
// reads the key's codes once and multiplies them with all rep query rows (float32 queries in
// shared memory, the group's scale and bias applied per group: s * sum(code * q) + b * sum(q)).
// Values: the tile's codes, scales and biases are staged in shared memory with 16-byte loads; 64
// threads x 2 key halves each own D / 64 output columns and accumulate p * (s * code + b).
// qattn_combine merges the splits (and the sink) and rounds to the output type.
#include "common.cuh"

namespace nvc {

constexpr int QA_THREADS = 128, QA_TILE = 128, QA_MAX_REP = 8;

struct QAttnParams {
    const void *q;                               // [B, Hq, 1, D]
    const uint32_t *kw, *vw;                     // codes
    const void *ks, *kb, *vs, *vb;               // scales, biases
    const void *sinks;                           // [Hq] or null
    float *part;                                 // [B, Hq, splits, D + 2]: acc, m, l
    void *out;                                   // [B, Hq, 1, D]
    int32_t B, Hq, Hkv, S, capacity, splits, chunk;
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
        qs[d][h] = h < rep ? __fmul_rn(DT<T>::load((const T *)p.q, ((size_t)b * p.Hq + hk * rep + h) * D + d), p.scale) : 0.0f;
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

template <typename T, int D>
__global__ void __launch_bounds__(D) qattn_combine_kernel(QAttnParams p) {
    const int h = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
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
    DT<T>::store((T *)p.out, ((size_t)b * p.Hq + h) * D + d, den > 0.0f ? __fdiv_rn(num, den) : 0.0f);
}

template <typename T, int BITS, int D>
static int32_t qattn_launch(nvc_device *dev, const QAttnParams &p, int gs) {
    dim3 grid((unsigned)p.splits, (unsigned)p.Hkv, (unsigned)p.B);
    if (gs == 32) qattn_split_kernel<T, BITS, D, 32><<<grid, QA_THREADS, 0, dev->stream>>>(p);
    else if (gs == 64) qattn_split_kernel<T, BITS, D, 64><<<grid, QA_THREADS, 0, dev->stream>>>(p);
    else if (D == 128) qattn_split_kernel<T, BITS, D, D == 128 ? 128 : 64><<<grid, QA_THREADS, 0, dev->stream>>>(p);
    NVC_TRY(check_launch(dev, "qattn_split_kernel"));
    qattn_combine_kernel<T, D><<<dim3((unsigned)p.Hq, (unsigned)p.B), D, 0, dev->stream>>>(p);
    return check_launch(dev, "qattn_combine_kernel");
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
                                           const void *v_biases, const void *sinks, int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t D,
                                           int64_t capacity, float scale, void *out) {
    NVC_TRY(make_current(dev));
    NVC_TRY(check_quant("quantized_attention", quant));
    if (quant->mode != NVC_AFFINE) return set_error(NVC_ERR_INVALID_ARGUMENT, "quantized_attention: keys and values need one affine quantization");
    const int bits = quant->bits, gs = quant->group_size;
    if (dtype != NVC_F16 && dtype != NVC_BF16 && dtype != NVC_F32) return set_error(NVC_ERR_UNSUPPORTED, "quantized_attention: unsupported dtype %d", dtype);
    if (B < 0 || Hq < 0 || Hkv < 0 || S < 0 || capacity < S) return set_error(NVC_ERR_INVALID_ARGUMENT, "quantized_attention: invalid shape");
    if ((D != 64 && D != 128) || (bits != 3 && bits != 4 && bits != 8) || D % gs != 0)
        return set_error(NVC_ERR_UNSUPPORTED, "quantized_attention: head size %lld with %d bits in groups of %d (64 or 128; 3, 4 or 8; a group within a head)",
                         (long long)D, bits, gs);
    if (B * Hq == 0) return NVC_OK;
    if (Hkv <= 0 || Hq % Hkv != 0) return set_error(NVC_ERR_INVALID_ARGUMENT, "quantized_attention: %lld query heads over %lld key heads", (long long)Hq, (long long)Hkv);
    const int64_t rep = Hq / Hkv;
    if (rep != 1 && rep != 2 && rep != 4 && rep != 8) return set_error(NVC_ERR_UNSUPPORTED, "quantized_attention: %lld query heads per key head (1, 2, 4 or 8)", (long long)rep);
    if (B > 65535 || Hkv > 65535 || S > INT32_MAX || capacity > INT32_MAX) return set_error(NVC_ERR_UNSUPPORTED, "quantized_attention: too long");
    if (!q || !out || (S > 0 && (!k_codes || !k_scales || !k_biases || !v_codes || !v_scales || !v_biases)))
        return set_error(NVC_ERR_INVALID_ARGUMENT, "quantized_attention: null operand");
    if (((uintptr_t)k_codes | (uintptr_t)v_codes) % 16 != 0) return set_error(NVC_ERR_UNSUPPORTED, "quantized_attention: the codes must be 16-byte aligned");
    if (dev->capturing) return set_error(NVC_ERR_UNSUPPORTED, "quantized_attention: not inside a recorded step (it takes scratch from the pool)");
    // splits: enough blocks to keep five on every multiprocessor (what their registers allow), whole tiles of 128 keys each
    const int64_t tiles = S > 0 ? (S + QA_TILE - 1) / QA_TILE : 1;
    int64_t splits = (5 * (int64_t)dev->prop.multiProcessorCount + B * Hkv - 1) / (B * Hkv);
    if (splits > tiles) splits = tiles;
    if (splits < 1) splits = 1;
    const int64_t chunk = (tiles + splits - 1) / splits * QA_TILE;
    splits = S > 0 ? (S + chunk - 1) / chunk : 1;
    void *part = nullptr;
    NVC_TRY(dev->pool.alloc((size_t)B * Hq * splits * (D + 2) * sizeof(float), &part));
    QAttnParams p{q, k_codes, v_codes, k_scales, k_biases, v_scales, v_biases, sinks, (float *)part, out,
                  (int32_t)B, (int32_t)Hq, (int32_t)Hkv, (int32_t)S, (int32_t)capacity, (int32_t)splits, (int32_t)chunk, scale};
    int32_t rc = dtype == NVC_F16 ? qattn_typed<__half>(dev, p, bits, (int)D, gs)
                 : dtype == NVC_BF16 ? qattn_typed<__nv_bfloat16>(dev, p, bits, (int)D, gs) : qattn_typed<float>(dev, p, bits, (int)D, gs);
    dev->pool.free(part);  // (the pool hands the block out again in stream order)
    return rc;
}
