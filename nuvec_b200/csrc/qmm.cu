// Many-row quantized products on the 5th-generation tensor cores (tcgen05), for prefill and
// for the grouped (sorted) mixture-of-experts product:
//
//     y[tok, n] = sum_k x[tok, k] * dequantize(w)[n, k]         (weights stored [N, K], "transposed")
//
// One persistent block per multiprocessor walks output tiles of 128 weight rows x BT tokens.
// The weight tile is the UMMA "A" operand (M = 128), the activations the "B" operand (N = BT):
// the accumulator D[128 x BT] (float32) lives in tensor memory, each dequantized weight is reused
// by BT tokens, and a group of few tokens (an expert with 32 rows) still fills all 128 lanes.
//
// Warp roles (768 threads):
//   warps 0-3   epilogue: tcgen05.ld the finished accumulator, round to bfloat16, store y
//   warp  4     TMA producer of activation tiles (64 k x BT tokens, 128-byte swizzle): the MMA's
//               B operand, read from shared memory
//   warp  6     TMA producer of packed weight slabs (128 rows x 128 bytes, 128-byte swizzle),
//               on its own ring so it runs ahead of the activation stages
//   warps 7-22  dequantizers (four groups of four warps take k-blocks in turn; thread = weight
//               row = tensor-memory lane): packed codes -> 64 bfloat16 in registers, with
//               exactly the reference's two roundings (crates/nuvec-core/src/kernels.rs:835-859),
//               so the tensor-core operands are bit-identical to the reference's dequantized
//               matrix -> tcgen05.st into the block's stage of tensor memory: the MMA's A
//               operand.  Dequantized weights never pass through shared memory, whose bandwidth
//               (operand reads + TMA writes + the dequantizers' traffic) bounded an earlier version.
//   warp  5     MMA issuer: 4 x tcgen05.mma.kind::f16 (K = 16, A from tensor memory) per 64-k
//               block; tcgen05.commit releases the stage / publishes the accumulator.  It waits
//               on hardware named barriers only
//   warp  23    watcher: waits on the mbarriers for the MMA warp and hands each full stage over
//               through a named barrier
// Tensor memory (512 columns): two accumulators of BT columns, then the weight ring of 32 columns
// per stage.
// Two accumulator buffers in tensor memory let the epilogue of one tile overlap the main loop
// of the next.  All waits are bounded: a wait that gives up raises an abort flag that every
// other wait observes, the block frees its tensor memory and returns, and the host reports the
// failure at the next synchronisation.
//
// Reference behaviour covered: MLX/nuvec's qmm_t, qmm_t_splitk, nax qmm_t and gather_qmm_rhs
// kernels (crates/nuvec-kernels/src/metal/quantized.h:1358-1485, 2388-2519, 3301-3449;
// nax/quantized.metal); CPU result crates/nuvec-core/src/kernels.rs:1091-1142 and, for the
// gather, crates/nuvec-core/src/quantized.rs:679-719.
#include "qmm.cuh"
#include "tcgen05.cuh"

#include <cuda.h>

#include <cstdlib>
#include <cstring>

namespace nvc {

// ── optional role timing (diagnostic builds only: -DNUVEC_TIMELINE) ─────────────────────────
// Every role of blocks 0 and 1 adds up the clock cycles it spends inside each of its waits (and
// in total); nvc_debug_qmm_timing (end of this file) fetches the sums of the last launch.
#ifdef NUVEC_TIMELINE
constexpr int QT_ROLES = 8, QT_SLOTS = 6;
__device__ long long g_qmm_timing[2][QT_ROLES][QT_SLOTS];
#define QT_BEGIN long long qt_[QT_SLOTS] = {0, 0, 0, 0, 0, 0}; const long long qt_start_ = clock64();
#define QT(k, ...) { const long long qt_t_ = clock64(); __VA_ARGS__; qt_[k] += clock64() - qt_t_; }
#define QT_END(role, writer)                                                        \
    if (blockIdx.x < 2 && (writer)) {                                               \
        qt_[0] = clock64() - qt_start_;                                             \
        for (int q_ = 0; q_ < QT_SLOTS; q_++) g_qmm_timing[blockIdx.x][role][q_] = qt_[q_]; \
    }
#else
#define QT_BEGIN
#define QT(k, ...) { __VA_ARGS__; }
#define QT_END(role, writer)
#endif

constexpr int QMM_BN = 128;  // weight rows per tile (UMMA M)
constexpr int QMM_BK = 64;   // k-values per block: one 128-byte swizzle row of bfloat16
constexpr int QMM_EPI_WARPS = 4, QMM_DQ_WARPS = 16, QMM_DQ_GROUPS = 4;  // dequantizers: groups of 4 warps
constexpr uint32_t QMM_EPI_BARRIER = 9;  // named barrier of the epilogue warps (1 .. 8 belong to the stages)
constexpr int QMM_WATCH_WARP = QMM_EPI_WARPS + 3 + QMM_DQ_WARPS;  // the warp that waits on behalf of the MMA warp
constexpr int QMM_THREADS = (QMM_WATCH_WARP + 1) * 32;
constexpr int QMM_W_STAGES = 2;          // packed-weight slabs in flight
constexpr uint32_t QMM_W_BYTES = 128 * 128;  // one slab: 128 rows x 128 bytes
constexpr int QMM_TABLE_BYTES = 4112;        // the grouped products' tables: 2 x (512 + 1) ints, rounded up to 16 bytes
constexpr int QMM_EPI_STAGE_BYTES = 4 * 2048;  // epilogue: 32 tokens x 32 weight rows of bfloat16 per warp

struct QmmKernelParams {
    const uint16_t *scales, *biases;  // bfloat16 [weight rows, K / gs]
    const uint8_t *fp_scales;         // uint8 codes for mxfp4 / nvfp4 (scales aliased), else nullptr
    const float *global;              // nvfp4 global scale(s) or nullptr
    uint16_t *y;                      // bfloat16 [rows, N]
    const int32_t *offsets;           // grouped: first row of each expert, else nullptr
    int32_t *error;                   // host-visible word: nonzero when a wait gave up
    float *partials;                  // [tail tiles][splits][BT tokens][128 rows] float32 (K-split tiles)
    uint32_t *counters;               // [tail tiles] arrivals, zero on entry and on exit
    int32_t full_waves, tail_tiles, splits, tail_rounds;  // the schedule, see Item
    int32_t experts, rows, N, K;
    int32_t gs_shift, row_groups, mode, expert_global;
};


// Instruction descriptor: D = f32, A = B = bf16, both K-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t umma_idesc(int n, int m = QMM_BN) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ uint32_t q_lop3(uint32_t a, uint32_t mask, uint32_t orv) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));
    return r;
}
__device__ __forceinline__ uint32_t q_prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
__device__ __forceinline__ uint32_t q_fma(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}
__device__ __forceinline__ uint32_t q_add(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t q_mul(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}

// ── dequantization of 32 k-values of one weight row into 64 bytes (4 chunks of 16) ─────────
// Affine, reference arithmetic: p = rn(code * scale), w = rn(p + bias), both in bfloat16.
// Codes enter as the bfloat16 number 128 + code (code bits ORed into the mantissa of 128.0);
// fma(128 + c, s, -128 s) is the single rounding of the exact product c * s.
struct Affine {
    uint32_t s2, ns2, b2;
    __device__ __forceinline__ uint32_t finish(uint32_t m) const { return q_add(q_fma(m, s2, ns2), b2); }
};
// 4 bits: word = 8 codes.  a = w, b = w >> 4: byte j of a has code 2j in its low nibble, byte j of
// b has code 2j+1 there; prmt gathers the two bytes into the two halves, lop3 masks and ORs 128.0.
__device__ __forceinline__ uint4 dequant_word4(uint32_t w, const Affine &q) {
    const uint32_t b = w >> 4;
    uint4 o;
    // selector: result byte 0 <- a.byte j, result byte 2 <- b.byte j (bytes 1 and 3 are masked away)
    o.x = q.finish(q_lop3(q_prmt(w, b, 0x0400u), 0x000F000Fu, 0x43004300u));
    o.y = q.finish(q_lop3(q_prmt(w, b, 0x0501u), 0x000F000Fu, 0x43004300u));
    o.z = q.finish(q_lop3(q_prmt(w, b, 0x0602u), 0x000F000Fu, 0x43004300u));
    o.w = q.finish(q_lop3(q_prmt(w, b, 0x0703u), 0x000F000Fu, 0x43004300u));
    return o;
}
// 8 bits: the byte is rebuilt exactly from its nibbles (16 * hi + lo <= 255 fits bfloat16), then
// multiplied and biased with one rounding each.  Two words (8 codes) make one 16-byte chunk.
__device__ __forceinline__ uint2 dequant_word8(uint32_t w, const Affine &q) {
    const uint32_t k16 = 0x41804180u, kn2048 = 0xC500C500u, kn128 = 0xC300C300u;
    const uint32_t h = w >> 4;
    uint2 o;
    {
        uint32_t lo = q_lop3(q_prmt(w, w, 0x0100u), 0x000F000Fu, 0x43004300u);   // codes 0, 1 (low nibbles)
        uint32_t hi = q_lop3(q_prmt(h, h, 0x0100u), 0x000F000Fu, 0x43004300u);   // their high nibbles
        uint32_t code = q_add(q_fma(hi, k16, kn2048), q_add(lo, kn128));
        o.x = q_add(q_mul(code, q.s2), q.b2);
    }
    {
        uint32_t lo = q_lop3(q_prmt(w, w, 0x0302u), 0x000F000Fu, 0x43004300u);   // codes 2, 3
        uint32_t hi = q_lop3(q_prmt(h, h, 0x0302u), 0x000F000Fu, 0x43004300u);
        uint32_t code = q_add(q_fma(hi, k16, kn2048), q_add(lo, kn128));
        o.y = q_add(q_mul(code, q.s2), q.b2);
    }
    return o;
}
// 2 bits: word = 16 codes; codes 2j, 2j+1 sit in bits [4j, 4j+4).
__device__ __forceinline__ void dequant_word2(uint32_t w, const Affine &q, uint4 &o0, uint4 &o1) {
    const uint32_t b = w >> 2;
    uint32_t r[8];
#pragma unroll
    for (int j = 0; j < 8; j++) {
        // byte j/2 holds codes 4(j/2) .. 4(j/2)+3; pair j = codes (2j, 2j+1): shift the byte pair by 4 (j odd)
        const uint32_t sel = 0x0400u + 0x0101u * (uint32_t)(j >> 1);
        uint32_t t = q_prmt(w, b, sel);
        if (j & 1) t >>= 4;
        r[j] = q.finish(q_lop3(t, 0x00030003u, 0x43004300u));
    }
    o0 = make_uint4(r[0], r[1], r[2], r[3]);
    o1 = make_uint4(r[4], r[5], r[6], r[7]);
}

// E2M1 code pairs -> bfloat16 pairs times the group scale.  The code's three magnitude bits become
// exponent[1:0] and mantissa[6] of a bfloat16 whose value is magnitude * 2^-126 (the subnormal
// codes 0 and 0.5 included); multiplying by 2^126 restores the value and multiplying by the
// scale (a power of two, or an E4M3 number with 4 significant bits) is exact: the product has at
// most 6 significant bits.  It equals the reference's float32 value scale * code
// (crates/nuvec-core/src/kernels.rs:976-1009).
__device__ __forceinline__ uint4 dequant_word_fp4(uint32_t w, uint32_t scale2) {
    const uint32_t b = w >> 4;
    uint32_t t[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const uint32_t p = q_prmt(w, b, 0x0400u + 0x0101u * (uint32_t)j);  // halves: codes 2j, 2j+1 in bits [3:0]
        const uint32_t bits = ((p & 0x00070007u) << 6) | ((p & 0x00080008u) << 12);
        t[j] = q_mul(q_mul(bits, 0x7E807E80u), scale2);
    }
    return make_uint4(t[0], t[1], t[2], t[3]);
}
// 8-bit floating point (mxfp8: E4M3 codes): the code's seven magnitude bits become exponent[3:0] and mantissa[6:4] of
// a bfloat16 (the value * 2^-120, subnormal codes as bfloat16 subnormals); times 2^120 and the scale (a power of two)
// it is the reference's float32 decode exactly.  The two NaN codes, which the reference's quantizer never writes, read
// as 480.  Halves: codes (0, 1) and (2, 3).
__device__ __forceinline__ uint2 dequant_word_fp8(uint32_t w, uint32_t scale2) {
    uint2 o;
    {
        const uint32_t x = q_prmt(w, w, 0x0100u);  // bytes 0, 1 in the low byte of each half
        o.x = q_mul(q_mul(q_lop3(x << 8, 0x80008000u, (x << 4) & 0x07F007F0u), 0x7B807B80u), scale2);
    }
    {
        const uint32_t x = q_prmt(w, w, 0x0302u);  // bytes 2, 3
        o.y = q_mul(q_mul(q_lop3(x << 8, 0x80008000u, (x << 4) & 0x07F007F0u), 0x7B807B80u), scale2);
    }
    return o;
}
// bfloat16 pair {s, s} of a scale code: E8M0 (2^(code - 127); code 0 decodes to a float32 subnormal
// that the reference flushes to zero) or E4M3.
__device__ __forceinline__ uint32_t fp_scale2(uint32_t code, bool e8m0) {
    uint32_t h;
    if (e8m0) h = code == 0u ? 0u : (code << 7);
    else h = __float_as_uint(ftz(e4m3_to_f32(code))) >> 16;
    return (h & 0xFFFFu) * 0x10001u;
}

template <int BITS> struct QmmBits;
template <> struct QmmBits<4> { static constexpr int KPS = 4; };  // 64-k blocks per 128-byte packed slab row
template <> struct QmmBits<8> { static constexpr int KPS = 2; };
template <> struct QmmBits<2> { static constexpr int KPS = 8; };

// Tile bookkeeping shared by the roles.
struct TileInfo {
    int n0;        // first weight row of the tile inside its matrix
    int wrow0;     // first row in the stacked [experts * N] weight / scale arrays
    int tok0;      // first token row of the tile
    int tok_end;   // tokens at or past this row are not stored
    int expert;
};

// Grouped products: the experts' first rows and the number of token tiles before each expert, kept
// in shared memory (filled once per block), so that finding a tile's expert is a binary search in
// shared memory and not a walk over global memory by every role at every tile.
constexpr int QMM_MAX_TABLE_EXPERTS = 512;
struct GroupTable {
    const int *off;    // [experts + 1] first row of each expert, then the row count; nullptr: no table
    const int *tiles;  // [experts + 1] token tiles before each expert, then the total
};

// `half`: -1, or the block's rank in a pair, whose tiles are 2 x 128 weight rows (ungrouped products only).
template <int BT>
__device__ __forceinline__ bool tile_info(const QmmKernelParams &p, const GroupTable &gt, int tile, int n_tiles, TileInfo &ti,
                                          int half = -1) {
    const int nt = tile % n_tiles, j = tile / n_tiles;
    ti.n0 = half < 0 ? nt * QMM_BN : (2 * nt + half) * QMM_BN;
    if (!p.offsets) {
        ti.expert = 0;
        ti.wrow0 = ti.n0;
        ti.tok0 = j * BT;
        ti.tok_end = p.rows;
        return ti.tok0 < p.rows;
    }
    if (gt.off) {
        if (j >= gt.tiles[p.experts]) return false;
        int lo = 0, hi = p.experts;  // the expert e with tiles[e] <= j < tiles[e + 1]
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (gt.tiles[mid] <= j) lo = mid; else hi = mid;
        }
        ti.expert = lo;
        ti.wrow0 = lo * p.N + ti.n0;
        ti.tok0 = gt.off[lo] + (j - gt.tiles[lo]) * BT;
        ti.tok_end = gt.off[lo + 1];
        return true;
    }
    // grouped: token tile j of the concatenation of every expert's tiles
    int seen = 0;
    for (int e = 0; e < p.experts; e++) {
        const int lo = p.offsets[e], hi = e + 1 < p.experts ? p.offsets[e + 1] : p.rows;
        const int tiles_e = (hi - lo + BT - 1) / BT;
        if (j < seen + tiles_e) {
            ti.expert = e;
            ti.wrow0 = e * p.N + ti.n0;
            ti.tok0 = lo + (j - seen) * BT;
            ti.tok_end = hi;
            return true;
        }
        seen += tiles_e;
    }
    return false;
}

// The schedule.  Every block first takes `full_waves` whole tiles (tile = block + wave * grid).  The
// tiles left over (fewer than blocks) are cut along K into `splits` parts of whole packed-weight
// slabs, one part per block, so that the last wave -- or a product with fewer tiles than
// multiprocessors -- still keeps every multiprocessor busy.  Parts leave float32 partial tiles in
// scratch; the block that arrives last adds them in part order and writes the result.
struct Item {
    int tile, kb0, kb1;  // k-blocks [kb0, kb1) of this tile
    int part, parts, slot;
    int round;           // which of the block's (at most two) parts of left-over tiles this is
};
// `worker` of `grid` workers: a block of the grid, or a pair of blocks.
template <int KPS>
__device__ __forceinline__ bool qmm_item(const QmmKernelParams &p, int kblocks, int j, Item &it, int worker, int grid) {
    if (j < p.full_waves) {
        it.tile = worker + j * grid;
        it.kb0 = 0; it.kb1 = kblocks; it.part = 0; it.parts = 1; it.slot = 0; it.round = 0;
        return true;
    }
    // the parts of the left-over tiles are dealt round-robin, at most tail_rounds per block
    it.round = j - p.full_waves;
    const int pi = worker + it.round * grid;
    if (it.round >= p.tail_rounds || pi >= p.tail_tiles * p.splits) return false;
    it.slot = pi / p.splits;
    it.part = pi % p.splits;
    it.parts = p.splits;
    it.tile = p.full_waves * grid + it.slot;
    const int slabs = (kblocks + KPS - 1) / KPS;  // the launch keeps splits <= slabs: no part is empty
    it.kb0 = slabs * it.part / p.splits * KPS;
    it.kb1 = min(slabs * (it.part + 1) / p.splits * KPS, kblocks);
    return true;
}

// Stages of the dequantized-weight ring in tensor memory: 32 columns each, in what the two
// accumulators leave of the 512 columns.
// PAIR: two blocks of a cluster share a tile of 2 x 128 weight rows x BT tokens; each keeps half of
// the tokens' activations in its shared memory (the stage is half as large) and one accumulator.
template <int BT, bool PAIR = false> struct QmmTmem {
    // Two accumulators (the epilogue of one tile overlaps the main loop of the next) while they
    // leave 128 columns for the weight ring; the widest tile keeps a single one.
    static constexpr int ACC_BUFS = 2 * BT + 128 <= 512 ? 2 : 1;
    static constexpr int XT = PAIR ? BT / 2 : BT;  // token rows of a stage in this block's shared memory
    static constexpr int ACC_COLS = ACC_BUFS * BT;
    static constexpr int A_COL0 = ACC_COLS;
    // ring depth: what the tensor-memory columns and the shared memory (activation stages beside
    // two packed-weight slabs) both allow, at most 8
    static constexpr int BY_TMEM = (512 - ACC_COLS) / 32;
    static constexpr int BY_SMEM = (227 * 1024 - 2048 - 8192 - QMM_EPI_STAGE_BYTES - 2 * 128 * 128) / (XT * 64 * 2);
    static constexpr int FIT = BY_TMEM < BY_SMEM ? (BY_TMEM < 8 ? BY_TMEM : 8) : (BY_SMEM < 8 ? BY_SMEM : 8);
    // a multiple of the dequantizer groups, so that a stage is always refilled by the same group
    static constexpr int STAGES = FIT / QMM_DQ_GROUPS * QMM_DQ_GROUPS;
    static_assert(STAGES >= QMM_DQ_GROUPS, "token tile too wide for the weight ring");
};

template <int BITS, int BT, int STAGES, int MODE /*0 affine, 1 mxfp4, 2 mxfp8, 3 nvfp4*/, bool PAIR = false>
__global__ void __launch_bounds__(QMM_THREADS, 1)
qmm_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w, QmmKernelParams p,
           int total_tiles, int n_tiles) {
    constexpr int KPS = QmmBits<BITS>::KPS;
    using Ring = QmmTmem<BT, PAIR>;
    constexpr int XT = Ring::XT;
    constexpr uint32_t X_BYTES = XT * QMM_BK * 2;
    constexpr int A_COL0 = Ring::A_COL0, ACC_BUFS = Ring::ACC_BUFS;
    static_assert(STAGES == Ring::STAGES, "activation stages in shared memory and weight stages in tensor memory form one ring");
    static_assert(!PAIR || ACC_BUFS == 1, "a pair keeps one accumulator");
    // A pair works as one: both blocks walk the same items; `half` is the block's rank in the pair
    // (its 128 of the tile's 256 weight rows, its half of the tile's tokens), -1 without pairs.
    const int half = PAIR ? (int)pair_rank() : -1;
    const bool leader = !PAIR || half == 0;
    const int worker = PAIR ? (int)blockIdx.x >> 1 : (int)blockIdx.x;
    const int workers = PAIR ? (int)gridDim.x >> 1 : (int)gridDim.x;
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment for the swizzled tiles
    uint8_t *smem = reinterpret_cast<uint8_t *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *xs = smem;                                   // [STAGES][BT x 128 B]
    uint8_t *ws = xs + STAGES * X_BYTES;                  // [QMM_W_STAGES][128 x 128 B]
    uint64_t *bars = reinterpret_cast<uint64_t *>(ws + QMM_W_STAGES * QMM_W_BYTES);
    // empty[s]: the MMAs that read activation stage s (shared memory) and weight stage s (tensor
    // memory) are done; the activation producer and the dequantizers both wait on it.
    uint64_t *xfull = bars, *afull = xfull + STAGES, *empty = afull + STAGES;
    uint64_t *wfull = empty + STAGES, *wempty = wfull + QMM_W_STAGES;
    uint64_t *accfull = wempty + QMM_W_STAGES, *accempty = accfull + 2;
    // Pairs: afull, accempty and pxfull of the FIRST block are the ones waited on; the second block's
    // dequantizers, epilogue and watcher arrive there (its activation stage has landed: pxfull).
    uint64_t *pxfull = accempty + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(pxfull + STAGES);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    volatile int *last_flag = abort_flag + 1;  // epilogue: this block arrived last at a K-split tile
    int *table = reinterpret_cast<int *>(bars) + 256;  // behind the 1 KB of barriers and flags: 2 x (experts + 1) ints
    uint8_t *epi_stage = reinterpret_cast<uint8_t *>(bars) + 1024 + QMM_TABLE_BYTES;  // [epilogue warp][32 tokens][32 rows] bfloat16

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kblocks = p.K / QMM_BK;

    if (tid == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(xfull + s, 1);
            mbar_init(afull + s, (PAIR ? 2 : 1) * QMM_DQ_WARPS / QMM_DQ_GROUPS);
            mbar_init(empty + s, 1);
            mbar_init(pxfull + s, 1);
        }
        for (int s = 0; s < QMM_W_STAGES; s++) {
            mbar_init(wfull + s, 1);
            mbar_init(wempty + s, QMM_DQ_WARPS);
        }
        for (int s = 0; s < 2; s++) {
            mbar_init(accfull + s, 1);
            mbar_init(accempty + s, (PAIR ? 2 : 1) * QMM_EPI_WARPS);
        }
        *abort_flag = 0;
        *last_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 5) {  // all of tensor memory: two accumulators and the dequantized-weight ring
        if (PAIR) {  // the same warp of both blocks
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "n"(512) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "n"(512) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    GroupTable gt{nullptr, nullptr};
    const bool tabled = p.offsets && p.experts <= QMM_MAX_TABLE_EXPERTS;
    if (tabled) {
        for (int e = tid; e <= p.experts; e += QMM_THREADS) table[e] = e < p.experts ? p.offsets[e] : p.rows;
    }
    tc_fence_before();
    __syncthreads();
    if (PAIR) pair_sync();  // the other block's barriers exist before anything arrives on them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (tabled) {
        int *tiles = table + QMM_MAX_TABLE_EXPERTS + 1;
        if (tid == 0) {
            int seen = 0;
            for (int e = 0; e < p.experts; e++) {
                tiles[e] = seen;
                seen += (table[e + 1] - table[e] + BT - 1) / BT;
            }
            tiles[p.experts] = seen;
        }
        __syncthreads();
        gt.off = table;
        gt.tiles = tiles;
    }

    if (warp == 4) {
        // ── TMA producer, activations: one 64-k x BT tile per stage ─────────────────────────
        if (lane == 0) {
            QT_BEGIN
            uint32_t it = 0;  // k-blocks issued so far
            bool ok = true;
            for (int j = 0; ok; j++) {
                Item item;
                if (!qmm_item<KPS>(p, kblocks, j, item, worker, workers)) break;
                TileInfo ti;
                if (!tile_info<BT>(p, gt, item.tile, n_tiles, ti, half)) continue;
                for (int kb = item.kb0; kb < item.kb1 && ok; kb++, it++) {
                    const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
                    QT(1, ok = mbar_wait(empty + s, ph ^ 1, abort_flag))
                    if (!ok) break;
                    mbar_expect_tx(xfull + s, X_BYTES);
                    tma_load_2d(xs + s * X_BYTES, &tmap_x, kb * QMM_BK, ti.tok0 + (PAIR ? half * XT : 0), xfull + s);
                }
            }
            QT_END(0, true)
        }
    } else if (warp == 6) {
        // ── TMA producer, packed weights: runs ahead on its own ring, so a slab's latency is
        //    never behind the activation stages ─────────────────────────────────────────────
        if (lane == 0) {
            uint32_t wit = 0;  // weight slabs issued so far
            bool ok = true;
            for (int j = 0; ok; j++) {
                Item item;
                if (!qmm_item<KPS>(p, kblocks, j, item, worker, workers)) break;
                TileInfo ti;
                if (!tile_info<BT>(p, gt, item.tile, n_tiles, ti, half)) continue;
                for (int kb = item.kb0; kb < item.kb1 && ok; kb += KPS, wit++) {
                    const uint32_t s = wit % QMM_W_STAGES, ph = (wit / QMM_W_STAGES) & 1;
                    ok = mbar_wait(wempty + s, ph ^ 1, abort_flag);
                    if (!ok) break;
                    mbar_expect_tx(wfull + s, QMM_W_BYTES);
                    tma_load_2d(ws + s * QMM_W_BYTES, &tmap_w, (kb / KPS) * 128, ti.wrow0, wfull + s);
                }
            }
        }
    } else if (warp == 5) {
        // ── MMA issuer: A (weights) from tensor memory, B (activations) from shared memory ──
        // Any shared-memory load (an mbarrier test included) issued by the thread that issues
        // tcgen05.mma was measured at ~270 cycles per round on the B200, more than four MMA issues;
        // a hardware named barrier costs ~30.  So this warp never reads shared memory: the watcher
        // warp waits on the mbarriers (stage full, accumulator drained) and passes each stage on
        // through named barrier 1 + stage.  All lanes walk the loop; lane 0 issues.
        constexpr uint32_t idesc = umma_idesc(BT, PAIR ? 2 * QMM_BN : QMM_BN);
        QT_BEGIN
        uint32_t tcount = 0, s = 0;
        const uint32_t empty0 = smem_u32(empty);
        const uint64_t bd0 = umma_desc(smem_u32(xs));
        // (pairs: the first block's warp issues for both; the second block's has nothing to do)
        for (int j = 0; leader; j++) {
            Item item;
            if (!qmm_item<KPS>(p, kblocks, j, item, worker, workers)) break;
            TileInfo ti;
            if (!tile_info<BT>(p, gt, item.tile, n_tiles, ti, half)) continue;
            const uint32_t buf = tcount % ACC_BUFS;
            const uint32_t d = tmem_base + buf * BT;
            for (int kb = item.kb0; kb < item.kb1; kb++) {
                QT(1, named_sync(1 + s))  // stage s is full (and, for kb = 0, the accumulator is drained)
                QT(2, if (lane == 0) {
                    tc_fence_after();
                    const uint32_t at = tmem_base + A_COL0 + s * 32;
                    const uint64_t bd = bd0 + (uint64_t)(s * (X_BYTES >> 4));
_Pragma("unroll")
                    for (int k = 0; k < QMM_BK / 16; k++) {  // 16 k-values: 8 columns of A, 32 bytes of the swizzle row of B
                        if (PAIR) tc_mma_bf16_ta_pair(d, at + 8 * k, bd + (uint64_t)(2 * k), idesc, kb != item.kb0 || k != 0);
                        else tc_mma_bf16_ta(d, at + 8 * k, bd + (uint64_t)(2 * k), idesc, kb != item.kb0 || k != 0);
                    }
                    // frees both halves of the stage (in both blocks of a pair) once these MMAs have read them
                    if (PAIR) tc_commit_pair(empty0 + 8 * s);
                    else tc_commit_addr(empty0 + 8 * s);
                })
                __syncwarp();
                if (++s == STAGES) s = 0;
            }
            if (lane == 0) {
                if (PAIR) tc_commit_pair(smem_u32(accfull + buf));
                else tc_commit(accfull + buf);
            }
            __syncwarp();
            tcount++;
        }
        QT_END(1, lane == 0)
    } else if (warp == QMM_WATCH_WARP) {
        // ── watcher: the MMA warp's eyes.  It arrives on the named barrier of every stage exactly
        //    once per k-block whatever happens (after a wait gave up it stops waiting, not
        //    arriving), so the MMA warp can never be left behind in a barrier. ──
        uint32_t tcount = 0, s = 0, ph = 0;
        bool ok = true;
        QT_BEGIN
        for (int j = 0;; j++) {
            Item item;
            if (!qmm_item<KPS>(p, kblocks, j, item, worker, workers)) break;
            TileInfo ti;
            if (!tile_info<BT>(p, gt, item.tile, n_tiles, ti, half)) continue;
            const uint32_t buf = tcount % ACC_BUFS, aph = (tcount / ACC_BUFS) & 1;
            if (!leader) {
                // second block of a pair: tells the first when this block's half of a stage has landed
                for (int kb = item.kb0; kb < item.kb1; kb++) {
                    QT(1, if (lane == 0 && ok) ok = mbar_wait(xfull + s, ph, abort_flag))
                    QT(2, if (lane == 0 && ok) mbar_arrive_leader(pxfull + s))
                    __syncwarp();
                    if (++s == STAGES) {
                        s = 0;
                        ph ^= 1;
                    }
                }
                tcount++;
                continue;
            }
            QT(4, if (lane == 0 && ok) ok = mbar_wait(accempty + buf, aph ^ 1, abort_flag))  // the epilogue has drained this buffer
            for (int kb = item.kb0; kb < item.kb1; kb++) {
                QT(1, if (lane == 0 && ok) ok = mbar_wait(xfull + s, ph, abort_flag))
                QT(2, if (PAIR && lane == 0 && ok) ok = mbar_wait(pxfull + s, ph, abort_flag))
                QT(3, if (lane == 0 && ok) ok = mbar_wait(afull + s, ph, abort_flag))
                __syncwarp();
                QT(5, named_arrive(1 + s))
                if (++s == STAGES) {
                    s = 0;
                    ph ^= 1;
                }
            }
            tcount++;
        }
        QT_END(2, lane == 0)
    } else if (warp >= 7 && warp < QMM_WATCH_WARP) {
        // ── dequantizers ─────────────────────────────────────────────────────────────────
        // Four groups of 4 warps take k-blocks in turn.  Thread = weight row = tensor-memory lane
        // (a warp reaches the 32 lanes of its rank in the warpgroup): it rebuilds the 64 k-values of
        // its row in registers and stores them as 32 columns of the block's stage, where the MMA
        // reads its A operand.  Nothing dequantized passes through shared memory.
        const int row = 32 * (warp & 3) + lane, group = (warp - 7) >> 2;
        const int sw = row & 7;  // swizzle phase of this row in the packed slab
        const uint32_t lane_base = (uint32_t)(32 * (warp & 3)) << 16;
        uint32_t it_base = 0, wit = 0;
        bool ok = true;
        QT_BEGIN
        // scale / bias codes of one block: [half] for 32-value halves (equal when the group is larger)
        auto load_consts = [&](const uint16_t *sc, const uint16_t *bi, const uint8_t *fsc, int kb, uint32_t (&sv)[2], uint32_t (&bv)[2]) {
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const int k = kb * QMM_BK + h * 32;
                if (MODE == 0) { sv[h] = sc[k >> p.gs_shift]; bv[h] = bi[k >> p.gs_shift]; }
                else { sv[h] = fsc[k >> p.gs_shift]; bv[h] = MODE == 3 ? fsc[(k + 16) >> p.gs_shift] : 0u; }
            }
        };
        for (int j = 0; ok; j++) {
            Item item;
            if (!qmm_item<KPS>(p, kblocks, j, item, worker, workers)) break;
            TileInfo ti;
            if (!tile_info<BT>(p, gt, item.tile, n_tiles, ti, half)) continue;
            // rows past N (last tile) read the last valid row's scales; their outputs are not stored
            const int wr = ti.wrow0 + min(row, p.N - 1 - ti.n0);
            const uint16_t *sc = p.scales + (size_t)wr * p.row_groups;
            const uint16_t *bi = p.biases ? p.biases + (size_t)wr * p.row_groups : nullptr;
            const uint8_t *fsc = p.fp_scales ? p.fp_scales + (size_t)wr * p.row_groups : nullptr;
            uint32_t s_next[2] = {0, 0}, b_next[2] = {0, 0};
            // this group's blocks are those at ring positions = group (mod groups): the same warps
            // always refill the same stages, so nobody is ever two phases ahead of a barrier
            const int first = item.kb0 + (group + QMM_DQ_GROUPS - (int)(it_base % QMM_DQ_GROUPS)) % QMM_DQ_GROUPS;
            if (first < item.kb1) load_consts(sc, bi, fsc, first, s_next, b_next);
            for (int slab = item.kb0 / KPS; slab * KPS < item.kb1 && ok; slab++, wit++) {
                const uint32_t wsi = wit % QMM_W_STAGES, wph = (wit / QMM_W_STAGES) & 1;
                bool have = false;
#pragma unroll 1
                for (int kq = 0; kq < KPS; kq++) {
                    const int kb = slab * KPS + kq;
                    if (kb >= item.kb1) break;
                    if ((int)((it_base + kb - item.kb0) % QMM_DQ_GROUPS) != group) continue;
                    const uint32_t s_cur[2] = {s_next[0], s_next[1]}, b_cur[2] = {b_next[0], b_next[1]};
                    if (kb + QMM_DQ_GROUPS < item.kb1) load_consts(sc, bi, fsc, kb + QMM_DQ_GROUPS, s_next, b_next);  // prefetch
                    if (!have) {
                        QT(1, ok = mbar_wait(wfull + wsi, wph, abort_flag))
                        have = true;
                    }
                    const uint8_t *wrow = ws + wsi * QMM_W_BYTES + row * 128;
                    uint32_t v[32];  // 64 bfloat16: column c of the stage holds k = 2c, 2c + 1
                    if (ok) {
                        Affine q[2];
                        uint32_t fa[2], fb[2];
#pragma unroll
                        for (int h = 0; h < 2; h++) {
                            if (MODE == 0) {
                                q[h].s2 = s_cur[h] * 0x10001u;
                                q[h].b2 = b_cur[h] * 0x10001u;
                                q[h].ns2 = q_mul(q[h].s2, 0xC300C300u);  // -128 s, exact
                            } else {
                                // mxfp4: one scale per 32 values; nvfp4: one per 16 (two per half)
                                fa[h] = fp_scale2(s_cur[h], MODE != 3);
                                fb[h] = MODE == 3 ? fp_scale2(b_cur[h], false) : fa[h];
                            }
                        }
                        if (BITS == 4) {
#pragma unroll
                            for (int h = 0; h < 2; h++) {
                                const uint4 pk = *reinterpret_cast<const uint4 *>(wrow + (((kq * 2 + h) ^ sw) << 4));
                                const uint32_t wv[4] = {pk.x, pk.y, pk.z, pk.w};
#pragma unroll
                                for (int j = 0; j < 4; j++) {
                                    const uint4 o = MODE == 0 ? dequant_word4(wv[j], q[h]) : dequant_word_fp4(wv[j], j < 2 ? fa[h] : fb[h]);
                                    v[16 * h + 4 * j] = o.x; v[16 * h + 4 * j + 1] = o.y;
                                    v[16 * h + 4 * j + 2] = o.z; v[16 * h + 4 * j + 3] = o.w;
                                }
                            }
                        } else if (BITS == 8) {
#pragma unroll
                            for (int c = 0; c < 4; c++) {
                                const uint4 pk = *reinterpret_cast<const uint4 *>(wrow + (((kq * 4 + c) ^ sw) << 4));
                                const uint32_t wv[4] = {pk.x, pk.y, pk.z, pk.w};
#pragma unroll
                                for (int j = 0; j < 4; j++) {
                                    const uint2 o = MODE == 0 ? dequant_word8(wv[j], q[c >> 1]) : dequant_word_fp8(wv[j], fa[c >> 1]);
                                    v[8 * c + 2 * j] = o.x; v[8 * c + 2 * j + 1] = o.y;
                                }
                            }
                        } else {
                            const uint4 pk = *reinterpret_cast<const uint4 *>(wrow + ((kq ^ sw) << 4));
                            const uint32_t wv[4] = {pk.x, pk.y, pk.z, pk.w};
#pragma unroll
                            for (int j = 0; j < 4; j++) {
                                uint4 o0, o1;
                                dequant_word2(wv[j], q[j >> 1], o0, o1);
                                v[8 * j] = o0.x; v[8 * j + 1] = o0.y; v[8 * j + 2] = o0.z; v[8 * j + 3] = o0.w;
                                v[8 * j + 4] = o1.x; v[8 * j + 5] = o1.y; v[8 * j + 6] = o1.z; v[8 * j + 7] = o1.w;
                            }
                        }
                    }
                    const uint32_t it = it_base + (uint32_t)(kb - item.kb0), sa = it % STAGES, pha = (it / STAGES) & 1;
                    QT(2, ok = ok && mbar_wait(empty + sa, pha ^ 1, abort_flag))  // the MMAs that read this stage are done
                    if (!ok) break;
                    QT(3, tc_fence_after();
                    tc_st32(tmem_base + lane_base + A_COL0 + sa * 32, v);
                    tc_st_wait();
                    tc_fence_before();  // the stores are ordered before the arrive the MMA thread waits on
                    __syncwarp())
                    QT(4, if (lane == 0) {
                        if (PAIR) mbar_arrive_leader(afull + sa);
                        else mbar_arrive(afull + sa);
                    })
                }
                // A warp none of whose blocks lay in this slab still waits for the slab before it
                // releases it: otherwise it could run ahead and its arrival for a later slab would
                // be counted into this one's phase.
                if (!have && ok) ok = mbar_wait(wfull + wsi, wph, abort_flag);
                __syncwarp();
                if (lane == 0) mbar_arrive(wempty + wsi);
            }
            it_base += (uint32_t)(item.kb1 - item.kb0);
        }
        QT_END(3 + group, (warp & 3) == 3 && lane == 0)
    } else {
        // ── epilogue: warp q owns tensor-memory lanes 32q .. 32q+31 = weight rows n0 + 32q + lane ──
        uint32_t tcount = 0;
        bool ok = true;
        QT_BEGIN
        for (int jj = 0; ok; jj++) {
            Item item;
            if (!qmm_item<KPS>(p, kblocks, jj, item, worker, workers)) break;
            TileInfo ti;
            if (!tile_info<BT>(p, gt, item.tile, n_tiles, ti, half)) continue;
            const uint32_t buf = tcount % ACC_BUFS, aph = (tcount / ACC_BUFS) & 1;
            // After a wait gave up the warp keeps walking the items without touching data: the
            // named barriers of K-split tiles below must still see all four epilogue warps.
            QT(1, if (ok) ok = mbar_wait(accfull + buf, aph, abort_flag))
            tc_fence_after();
            const int r = warp * 32 + lane;  // row of the tile
            const int n = ti.n0 + r;
            float gmul = 1.0f;
            if (MODE != 0 && p.global) gmul = (p.expert_global ? p.global[ti.expert] : p.global[0]) / (448.0f * 6.0f);
            if (item.parts == 1) {
                // Thread = weight row, registers = 32 tokens, but y is [token][row]: the warp turns each
                // 32 x 32 piece around in shared memory ([token][row], 64 bytes per token) and stores it
                // as 16-byte pieces of 8 rows -- 4 store instructions per piece instead of 32.  Rows in
                // whole groups of 8 (N a multiple of 8 and y aligned): otherwise element by element.
                const bool wide = (p.N & 7) == 0 && ((uintptr_t)p.y & 15) == 0;
                uint8_t *mine = epi_stage + warp * 2048;
                const int t8 = lane >> 2, g8 = lane & 3;  // this lane's token (of 8 per pass) and group of 8 rows
#pragma unroll 1
                for (int c = 0; c < BT / 32 && ok; c++) {
                    uint32_t v[32];
                    QT(2, tc_ld32(tmem_base + ((uint32_t)(warp * 32) << 16) + buf * BT + c * 32, v);
                    tc_ld_wait())
                    if (wide) {
                        if (ti.tok0 + c * 32 >= ti.tok_end) continue;  // (the whole warp: nothing of this piece is stored)
                        QT(3, _Pragma("unroll")
                        for (int j = 0; j < 32; j++) {
                            float f = __uint_as_float(v[j]);
                            if (MODE != 0) f *= gmul;
                            *reinterpret_cast<uint16_t *>(mine + j * 64 + lane * 2) = __bfloat16_as_ushort(__float2bfloat16_rn(f));
                        }
                        __syncwarp())
                        const int ng = ti.n0 + warp * 32 + g8 * 8;
                        uint16_t *dst = p.y + (size_t)(ti.tok0 + c * 32 + t8) * p.N + ng;
                        QT(4, _Pragma("unroll")
                        for (int i = 0; i < 4; i++) {
                            const uint4 q = *reinterpret_cast<const uint4 *>(mine + (i * 8 + t8) * 64 + g8 * 16);
                            if (ng < p.N && ti.tok0 + c * 32 + i * 8 + t8 < ti.tok_end)
                                *reinterpret_cast<uint4 *>(dst + (size_t)(i * 8) * p.N) = q;
                        }
                        __syncwarp())  // the piece has been read before the next one overwrites it
                    } else if (n < p.N) {
#pragma unroll
                        for (int j = 0; j < 32; j++) {
                            const int tok = ti.tok0 + c * 32 + j;
                            if (tok < ti.tok_end) {
                                float f = __uint_as_float(v[j]);
                                if (MODE != 0) f *= gmul;
                                p.y[(size_t)tok * p.N + n] = __bfloat16_as_ushort(__float2bfloat16_rn(f));
                            }
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    if (PAIR) mbar_arrive_leader(accempty + buf);
                    else mbar_arrive(accempty + buf);
                }
            } else {
                // One part of a tile cut along K: the float32 partial goes to scratch as
                // [token][row] (a warp writes 128 consecutive bytes per token); the block that
                // arrives last adds the parts in part order and rounds once.
                const int pslot = PAIR ? 2 * item.slot + half : item.slot;  // each block of a pair keeps its own rows' parts
                float *mine = p.partials + ((size_t)pslot * item.parts + item.part) * (size_t)(BT * QMM_BN);
#pragma unroll 1
                for (int c = 0; c < BT / 32 && ok; c++) {
                    uint32_t v[32];
                    tc_ld32(tmem_base + ((uint32_t)(warp * 32) << 16) + buf * BT + c * 32, v);
                    tc_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; j++)
                        if (ti.tok0 + c * 32 + j < ti.tok_end) __stcg(mine + (size_t)(c * 32 + j) * QMM_BN + r, __uint_as_float(v[j]));
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {  // the accumulator is free again
                    if (PAIR) mbar_arrive_leader(accempty + buf);
                    else mbar_arrive(accempty + buf);
                }
                __threadfence();
                named_sync_n(QMM_EPI_BARRIER, QMM_EPI_WARPS * 32);
                if (tid == 0) {
                    bool last = false;
                    if (ok) {
                        const uint32_t arrived = atomicAdd(p.counters + pslot, 1u);
                        last = arrived == (uint32_t)item.parts - 1;
                        if (last) p.counters[pslot] = 0u;  // rearmed for the next launch
                    }
                    // K-split parts are a block's last items: the whole block adds the parts up
                    // after its roles have finished (below).
                    if (last) *last_flag = *last_flag | (1 << item.round);
                }
            }
            tcount++;
        }
        QT_END(7, warp == 0 && lane == 0)
    }

    // ── teardown ────────────────────────────────────────────────────────────────────────
    tc_fence_before();
    __syncthreads();
    if (tid == 0 && *abort_flag && p.error) *p.error = 1;
    for (int round = 0; round < p.tail_rounds && !*abort_flag; round++) {
        if (!(*last_flag & (1 << round))) continue;
        // This block arrived last at this K-split tile: all its threads add the float32 parts in
        // part order (the sum does not depend on who arrived when), round once and store.
        Item item;
        TileInfo ti;
        if (qmm_item<KPS>(p, kblocks, p.full_waves + round, item, worker, workers) && tile_info<BT>(p, gt, item.tile, n_tiles, ti, half)) {
            __threadfence();
            float gmul = 1.0f;
            if (MODE != 0 && p.global) gmul = (p.expert_global ? p.global[ti.expert] : p.global[0]) / (448.0f * 6.0f);
            const int pslot = PAIR ? 2 * item.slot + half : item.slot;
            const float4 *base = reinterpret_cast<const float4 *>(p.partials + (size_t)pslot * item.parts * (size_t)(BT * QMM_BN));
            constexpr int TILE4 = BT * QMM_BN / 4;  // float4 per part
            const int tokens = min(BT, ti.tok_end - ti.tok0);
            for (int idx = tid; idx < tokens * (QMM_BN / 4); idx += QMM_THREADS) {
                const int t = idx / (QMM_BN / 4), r4 = idx % (QMM_BN / 4);
                float4 acc = __ldcg(base + idx);
                for (int q = 1; q < item.parts; q++) {
                    const float4 v = __ldcg(base + (size_t)q * TILE4 + idx);
                    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
                }
                const float f[4] = {acc.x, acc.y, acc.z, acc.w};
                const int n = ti.n0 + 4 * r4;
                uint16_t *dst = p.y + (size_t)(ti.tok0 + t) * p.N + n;
#pragma unroll
                for (int e = 0; e < 4; e++)
                    if (n + e < p.N) dst[e] = __bfloat16_as_ushort(__float2bfloat16_rn(MODE != 0 ? f[e] * gmul : f[e]));
            }
        }
    }
    if (PAIR) {
        // neither block leaves (or frees the pair's tensor memory) while the other may still arrive on its barriers
        tc_fence_before();
        pair_sync();
    }
    if (warp == 5) {
        tc_fence_after();
        if (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "n"(512) : "memory");
        else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "n"(512) : "memory");
    }
}


// ── host side ──────────────────────────────────────────────────────────────────────────────

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return (EncodeTiledFn)p;
    }();
    return fn;
}

// 2-D tensor map: `inner` elements per row (contiguous), `rows` rows `pitch_bytes` apart.
static int32_t make_map(CUtensorMap *map, CUtensorMapDataType type, const void *base, uint64_t inner, uint64_t rows,
                        uint64_t pitch_bytes, uint32_t box_inner, uint32_t box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return set_error(NVC_ERR_DRIVER, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {inner, rows}, strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {box_inner, box_rows}, estr[2] = {1, 1};
    CUresult r = fn(map, type, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error(NVC_ERR_DRIVER, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    return NVC_OK;
}

bool qmm_eligible(int32_t mode, int32_t gs, int32_t bits, int32_t dtype, int32_t transpose, int64_t M, int64_t N,
                  int64_t K, const void *x, int64_t ldx, const uint32_t *w) {
    (void)gs;
    static const bool disabled = getenv("NUVEC_QMM_DISABLE") != nullptr;  // read once: products then take the other kernels
    if (disabled) return false;
    if (dtype != NVC_BF16 || !transpose) return false;
    if (mode == NVC_AFFINE) {
        if (bits != 2 && bits != 4 && bits != 8) return false;
    } else if (mode == NVC_MXFP8) {
        if (bits != 8) return false;
    } else if (mode != NVC_MXFP4 && mode != NVC_NVFP4) {
        return false;
    }
    if (M < 1 || N < 1 || K < QMM_BK || K % QMM_BK != 0) return false;
    if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) return false;
    // TMA: 16-byte aligned bases and row pitches
    if ((uintptr_t)x % 16 != 0 || (ldx * 2) % 16 != 0) return false;
    if ((uintptr_t)w % 16 != 0 || (K * bits / 8) % 16 != 0) return false;
    return true;
}

// Scratch of the K-split tiles: float32 partial tiles and their arrival counters, owned by the
// device handle (kept apart from the few-row kernel's scratch, which a gather may be using for
// its expert offsets at the same time).  Counters are zero between launches.
static int32_t ensure_qmm_scratch(nvc_device *dev, size_t bytes, size_t counters) {
    if (dev->qmm_partials_bytes < bytes) {
        NVC_CUDA(cudaStreamSynchronize(dev->stream));
        if (dev->qmm_partials) dev->pool.free(dev->qmm_partials);
        dev->qmm_partials = nullptr;
        dev->qmm_partials_bytes = 0;
        NVC_TRY(dev->pool.alloc(bytes, &dev->qmm_partials));
        dev->qmm_partials_bytes = bytes;
    }
    if (dev->qmm_counters_len < counters) {
        NVC_CUDA(cudaStreamSynchronize(dev->stream));
        if (dev->qmm_counters) dev->pool.free(dev->qmm_counters);
        dev->qmm_counters = nullptr;
        dev->qmm_counters_len = 0;
        const size_t len = counters < 256 ? 256 : counters;
        void *ptr = nullptr;
        NVC_TRY(dev->pool.alloc(len * sizeof(uint32_t), &ptr));
        NVC_CUDA(cudaMemsetAsync(ptr, 0, len * sizeof(uint32_t), dev->stream));
        dev->qmm_counters = (uint32_t *)ptr;
        dev->qmm_counters_len = len;
    }
    return NVC_OK;
}

// PAIR: the grid is made of clusters of two blocks that work on tiles of 256 weight rows as one
// (`total_tiles`, `n_tiles` then count such tiles and `sms` below counts pairs).
template <int BITS, int BT, int MODE, bool PAIR = false>
static int32_t launch_cfg(nvc_device *dev, const CUtensorMap &mx, const CUtensorMap &mw, const QmmKernelParams &kp,
                          int total_tiles, int n_tiles) {
    constexpr uint32_t X_BYTES = QmmTmem<BT, PAIR>::XT * QMM_BK * 2;
    // one ring: activation stages in shared memory, weight stages in tensor memory
    constexpr int STAGES = QmmTmem<BT, PAIR>::STAGES;
    static_assert(8 * (QMM_MAX_TABLE_EXPERTS + 1) <= QMM_TABLE_BYTES, "the tables' area");
    // alignment slack, activation stages, packed-weight slabs, 1 KB of barriers and flags, the grouped products' tables,
    // the epilogue's staging area
    constexpr size_t smem = 1024 + STAGES * X_BYTES + QMM_W_STAGES * QMM_W_BYTES + 1024 + QMM_TABLE_BYTES + QMM_EPI_STAGE_BYTES;
    static_assert(smem <= 227 * 1024, "not enough shared memory for the pipeline");
    auto kernel = qmm_kernel<BITS, BT, STAGES, MODE, PAIR>;
    // the opt-in to this much dynamic shared memory is a per-device attribute of the instantiation
    static bool configured[64] = {};
    static std::mutex configured_mu;
    if (dev->ordinal < 0 || dev->ordinal >= 64) return set_error(NVC_ERR_UNSUPPORTED, "qmm: device ordinal %d", dev->ordinal);
    {
        std::lock_guard<std::mutex> g(configured_mu);
        if (!configured[dev->ordinal]) {
            NVC_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            configured[dev->ordinal] = true;
        }
    }
    // The schedule (see Item): whole tiles wave by wave, then the left-over tiles cut along K.
    QmmKernelParams k = kp;
    int sms = dev->prop.multiProcessorCount;
    if (PAIR) {
        // pairs that can be resident together (a pair needs two multiprocessors of one cluster-capable group)
        static int pairs[64] = {};
        std::lock_guard<std::mutex> g(configured_mu);
        if (pairs[dev->ordinal] == 0) {
            cudaLaunchConfig_t probe = {};
            probe.gridDim = dim3(2 * (unsigned)sms);
            probe.blockDim = dim3(QMM_THREADS);
            probe.dynamicSmemBytes = smem;
            cudaLaunchAttribute attr;
            attr.id = cudaLaunchAttributeClusterDimension;
            attr.val.clusterDim.x = 2;
            attr.val.clusterDim.y = attr.val.clusterDim.z = 1;
            probe.attrs = &attr;
            probe.numAttrs = 1;
            int n = 0;
            NVC_CUDA(cudaOccupancyMaxActiveClusters(&n, kernel, &probe));
            if (n < 1) return set_error(NVC_ERR_DRIVER, "qmm: no cluster of two blocks fits the device");
            pairs[dev->ordinal] = n < sms / 2 ? n : sms / 2;
        }
        sms = pairs[dev->ordinal];
    }
    const int kblocks = k.K / QMM_BK, slabs = (kblocks + QmmBits<BITS>::KPS - 1) / QmmBits<BITS>::KPS;
    int grid = sms < total_tiles ? sms : total_tiles;
    k.full_waves = total_tiles / grid;
    k.tail_tiles = total_tiles % grid;
    k.splits = 1;
    k.tail_rounds = 1;
    if (total_tiles < sms) {  // fewer tiles than multiprocessors: all of them are "left over"
        k.full_waves = 0;
        k.tail_tiles = total_tiles;
    }
    if (k.tail_tiles > 0) {
        // Parts per tile: whatever makes the left-over tiles finish soonest when the parts are dealt
        // over the multiprocessors in one or two rounds (time ~ rounds / parts, plus a little for
        // the partial sums); at least two slabs of weights per part, at most 16 parts.
        int best = 1;
        double best_cost = 1.0;
        for (int s2 = 2; s2 <= 16 && s2 <= slabs / 2; s2++) {
            const int rounds = (k.tail_tiles * s2 + sms - 1) / sms;
            if (rounds > 2) break;
            const double cost = (double)rounds / s2 + 0.05;
            if (cost < best_cost - 1e-9) {
                best_cost = cost;
                best = s2;
            }
        }
        k.splits = best;
        k.tail_rounds = (k.tail_tiles * best + sms - 1) / sms;
    }
    if (k.full_waves == 0) grid = k.tail_tiles * k.splits < sms ? k.tail_tiles * k.splits : sms;
    if (k.splits > 1) {
        const size_t blocks_per_tile = PAIR ? 2 : 1;  // each block of a pair keeps the parts of its own rows
        const size_t need = blocks_per_tile * k.tail_tiles * k.splits * BT * QMM_BN * sizeof(float);
        NVC_TRY(ensure_qmm_scratch(dev, need, blocks_per_tile * k.tail_tiles));
        k.partials = (float *)dev->qmm_partials;
        k.counters = dev->qmm_counters;
    }
    if (PAIR) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * (unsigned)grid);
        cfg.blockDim = dim3(QMM_THREADS);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = dev->stream;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2;
        attr.val.clusterDim.y = attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        NVC_CUDA(cudaLaunchKernelEx(&cfg, kernel, mx, mw, k, total_tiles, n_tiles));
    } else {
        kernel<<<grid, QMM_THREADS, smem, dev->stream>>>(mx, mw, k, total_tiles, n_tiles);
    }
    return check_launch(dev, "qmm_kernel");
}

template <int BITS, int MODE>
static int32_t launch_bt(nvc_device *dev, int bt, bool pair, const CUtensorMap &mx, const CUtensorMap &mw, const QmmKernelParams &kp,
                         int total_tiles, int n_tiles) {
    if (pair) return launch_cfg<BITS, 256, MODE, true>(dev, mx, mw, kp, total_tiles, n_tiles);
    switch (bt) {
    case 32: return launch_cfg<BITS, 32, MODE>(dev, mx, mw, kp, total_tiles, n_tiles);
    case 64: return launch_cfg<BITS, 64, MODE>(dev, mx, mw, kp, total_tiles, n_tiles);
    case 128: return launch_cfg<BITS, 128, MODE>(dev, mx, mw, kp, total_tiles, n_tiles);
    case 192: return launch_cfg<BITS, 192, MODE>(dev, mx, mw, kp, total_tiles, n_tiles);
    default: return launch_cfg<BITS, 256, MODE>(dev, mx, mw, kp, total_tiles, n_tiles);
    }
}

int32_t launch_qmm(nvc_device *dev, const QmmParams &p) {
    if (p.rows == 0 || p.N == 0) return NVC_OK;
    const int64_t experts = p.offsets ? p.experts : 1;
    // Token tile: the largest that the rows (per expert, on average) fill reasonably.
    const int64_t per = p.offsets ? (p.rows + experts - 1) / experts : p.rows;
    // 256 tokens keep one accumulator in tensor memory (the epilogue then stalls the MMAs for a
    // few per cent of a tile, which the wider MMA more than pays for); narrower tiles keep two.
    int bt = per > 192 ? 256 : per > 128 ? 192 : per > 64 ? 128 : per > 32 ? 64 : 32;
    // Experts' row counts scatter around the average, and a second token tile dequantizes the
    // expert's weights a second time (the kernel's cost is the dequantization, not the MMA
    // width): size the tile for the average plus half.
    // measured: 8-bit weights at 2048 rows run 294 us with 192-token tiles and 333-356 us with 256
    if (p.bits == 8 && per > 192 && per <= 4096) bt = 192;
    if (p.offsets) bt = per > 170 ? 256 : per > 128 ? 192 : per > 85 ? 192 : per > 42 ? 128 : per > 21 ? 64 : 32;
    // Pairs of blocks on tiles of 256 weight rows: ungrouped products of 256-token tiles whose rows
    // split evenly, with enough tiles to occupy the pairs.
    // Off unless NUVEC_QMM_PAIRS is set: measured 10-15 % slower than single blocks (the pair's
    // cross-block arrivals and its third wait per k-block cost more than the halved operand traffic gains).
    static const bool pairs_on = getenv("NUVEC_QMM_PAIRS") != nullptr;
    const bool pair = pairs_on && !p.offsets && bt == 256 && p.N % (2 * QMM_BN) == 0 &&
                      (p.N / (2 * QMM_BN)) * ((p.rows + bt - 1) / bt) >= dev->prop.multiProcessorCount / 2;
    const int n_tiles = pair ? (int)(p.N / (2 * QMM_BN)) : (int)((p.N + QMM_BN - 1) / QMM_BN);
    int64_t token_tiles;
    if (p.offsets) token_tiles = (p.rows + bt - 1) / bt + experts;  // upper bound: one partial tile per expert
    else token_tiles = (p.rows + bt - 1) / bt;
    const int64_t total = token_tiles * n_tiles;
    if (total > INT32_MAX) return set_error(NVC_ERR_UNSUPPORTED, "qmm: too many tiles");

    CUtensorMap mx, mw;
    NVC_TRY(make_map(&mx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, p.x, (uint64_t)p.K, (uint64_t)p.rows, (uint64_t)p.ldx * 2,
                     QMM_BK, (uint32_t)(pair ? bt / 2 : bt)));
    const uint64_t wrow_bytes = (uint64_t)p.K * p.bits / 8;
    NVC_TRY(make_map(&mw, CU_TENSOR_MAP_DATA_TYPE_UINT8, p.w, wrow_bytes, (uint64_t)(experts * p.N), wrow_bytes, 128, 128));

    NVC_TRY(ensure_error_word(dev));
    QmmKernelParams kp{};
    const bool affine = p.mode == NVC_AFFINE;
    kp.scales = affine ? (const uint16_t *)p.scales : nullptr;
    kp.biases = affine ? (const uint16_t *)p.biases : nullptr;
    kp.fp_scales = affine ? nullptr : (const uint8_t *)p.scales;
    kp.global = p.global;
    kp.y = (uint16_t *)p.y;
    kp.offsets = p.offsets;
    kp.error = dev->error_word_dev;
    kp.experts = (int32_t)experts;
    kp.rows = (int32_t)p.rows;
    kp.N = (int32_t)p.N;
    kp.K = (int32_t)p.K;
    kp.gs_shift = p.gs == 16 ? 4 : p.gs == 32 ? 5 : p.gs == 64 ? 6 : 7;
    kp.row_groups = (int32_t)(p.K / p.gs);
    kp.mode = p.mode;
    kp.expert_global = p.expert_global;
    const int tt = (int)total;
    if (affine) {
        switch (p.bits) {
        case 4: return launch_bt<4, 0>(dev, bt, pair, mx, mw, kp, tt, n_tiles);
        case 8: return launch_bt<8, 0>(dev, bt, pair, mx, mw, kp, tt, n_tiles);
        default: return launch_bt<2, 0>(dev, bt, pair, mx, mw, kp, tt, n_tiles);
        }
    }
    if (p.mode == NVC_MXFP8) return launch_bt<8, 2>(dev, bt, pair, mx, mw, kp, tt, n_tiles);
    if (p.mode == NVC_MXFP4) return launch_bt<4, 1>(dev, bt, pair, mx, mw, kp, tt, n_tiles);
    return launch_bt<4, 3>(dev, bt, pair, mx, mw, kp, tt, n_tiles);
}

}  // namespace nvc

#ifdef NUVEC_TIMELINE
// Diagnostic build only: cycles per role of blocks 0 and 1 in the last launch of the tensor-core
// kernel.  out[block][role][slot]: roles 0 activation producer, 1 MMA issuer, 2 watcher, 3-6 the
// dequantizer groups, 7 epilogue; slot 0 the role's total, the others its waits in program order.
extern "C" int32_t nvc_debug_qmm_timing(long long *out) {
    if (cudaDeviceSynchronize() != cudaSuccess ||
        cudaMemcpyFromSymbol(out, nvc::g_qmm_timing, sizeof(long long) * 2 * nvc::QT_ROLES * nvc::QT_SLOTS) != cudaSuccess)
        return NVC_ERR_DRIVER;
    return NVC_OK;
}
#endif
