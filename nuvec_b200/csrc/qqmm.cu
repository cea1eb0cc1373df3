// qqmm: the product of two operands that are BOTH quantized to NVFP4 (4-bit E2M1 codes, one E4M3
// scale per 16 values) or both to MXFP4 (one E8M0 scale per 32) on the tensor cores' native
// block-scaled path,
//
//     y[tok, n] = sum_k q(x)[tok, k] * w[n, k]
//
// where q(x) is x through its NVFP4 quantization (the reference's qqmm: fake_quant(x) followed by
// the ordinary quantized product, crates/nuvec-core/src/products.rs:337-352, 317-324).  Both
// operands reach the MMA as packed 4-bit codes with their scale factors:
//
//   tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16  D(tmem), A(smem), B(smem), SFA(tmem), SFB(tmem)
//   tcgen05.mma.cta_group::1.kind::mxf4.block_scale.block32      (MXFP4: two scales per row and MMA; a piece
//                                                                 of four serves two MMAs, the second through
//                                                                 scale-factor id 2 = byte 2 of the column)
//
// A block of 16 codes times 16 codes sums exactly in float32 (products of two 2-bit significands),
// and so does the block sum times the two E4M3 scales (8 more significant bits); only the order in
// which the blocks are added differs from the reference's float32 product of the dequantized
// operands, so the results agree within one output rounding -- unlike a product of bfloat16
// activations forced onto this path, which the reference does not define.
//
// Pipeline per call: quantize x (the kernel of quantize.cu, the reference's bits), lay the two scale
// arrays out the way the tensor core reads them (below), then the product kernel: one block per
// 128 weight rows x BN tokens, a TMA producer thread, an MMA thread and four epilogue warps.
//
// Scale-factor layout.  For one MMA (128 rows, 64 k-values = 4 scales per row) the tensor core reads
// four 32-bit columns of tensor memory: lane r % 32 of EVERY 32-lane quarter, column r / 32, byte s
// holds the scale of row r, k-block s.  The arrays of the reference ([rows, K / 16], one byte per
// scale) are re-laid-out into 512-byte pieces in that order -- byte (r % 32) * 16 + (r / 32) * 4 + s,
// [row tile of 128][k-block of 256][4 pieces] -- so that a stage's scales are one contiguous 2 KB
// bulk copy and a lane's four columns of a piece are one 16-byte shared-memory load.
//
// How the scales reach tensor memory.  tcgen05.cp (32x128b.warpx4) would do it, but it runs in the
// same in-order queue as the MMAs and, measured here, costs about as much as a quarter of an MMA
// whatever its shape; with three per MMA (one for the weights' scales, two for 256 tokens') the tensor
// pipe sat idle more than half of the main loop.  Instead the four epilogue warps, idle until the
// accumulator is complete, carry them: each warp owns one 32-lane quarter of tensor memory, reads a
// stage's pieces from shared memory and writes them to its quarter with tcgen05.st, into the stage's
// own set of scale columns, and signals the MMA thread.  The MMA queue holds MMAs only.
#include "common.cuh"
#include "tcgen05.cuh"

#include <cstring>

namespace nvc {

constexpr int QQ_BM = 128;        // weight rows per tile (UMMA M)
constexpr int QQ_KB = 256;        // k-values per stage: one 128-byte swizzle row of packed codes
constexpr int QQ_STEP = 64;       // k-values per MMA
constexpr int QQ_STAGES = 4;
constexpr int QQ_THREADS = 192;   // warp 0 TMA, warp 1 MMA + tensor memory, warps 2-5 epilogue
// 512-byte scale pieces (128 rows x 4 scales) per 128 rows and stage: 4 with a scale per 16 values, 2 per 32
__host__ __device__ constexpr int qq_pieces(int vs) { return QQ_KB / vs / 4; }

// [rows, K / vs] scale bytes -> the tensor core's pieces (see above); rows and k-blocks past the
// ends are zero (a zero scale times the zero codes TMA fills in).  One thread per 16 bytes of a
// piece: the four scales of one MMA step for rows r, r + 32, r + 64, r + 96.
__global__ void __launch_bounds__(256) qq_scale_layout_kernel(const uint8_t *__restrict__ scales, int64_t rows, int64_t per_row,
                                                              uint8_t *__restrict__ out, int64_t row_tiles, int64_t kblocks, int pieces) {
    const int64_t at = (int64_t)blockIdx.x * 256 + threadIdx.x;  // index of the 16-byte unit
    const int64_t total = row_tiles * kblocks * pieces * 32;
    if (at >= total) return;
    const int64_t piece = at >> 5, m0 = at & 31;
    const int64_t step = piece % pieces, kb = (piece / pieces) % kblocks, rt = piece / (pieces * kblocks);
    const int64_t s0 = (kb * pieces + step) * 4;
    uint32_t words[4];
#pragma unroll
    for (int m1 = 0; m1 < 4; m1++) {
        const int64_t r = rt * 128 + m1 * 32 + m0;
        uint32_t w = 0;
        if (r < rows) {
            const uint8_t *src = scales + r * per_row + s0;
            if (s0 + 4 <= per_row && ((uintptr_t)src & 3) == 0) {
                w = *reinterpret_cast<const uint32_t *>(src);
            } else {
#pragma unroll
                for (int b = 0; b < 4; b++)
                    if (s0 + b < per_row) w |= (uint32_t)src[b] << (8 * b);
            }
        }
        words[m1] = w;
    }
    reinterpret_cast<uint4 *>(out)[at] = make_uint4(words[0], words[1], words[2], words[3]);
}

// four 32-bit columns of the executing warp's quarter of tensor memory, one value per lane and column
__device__ __forceinline__ void qq_st4(uint32_t taddr, const uint4 &v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
template <int VS>
__device__ __forceinline__ void qq_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                       uint32_t accumulate) {
    if (VS == 16)
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
            ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb) : "memory");
    else
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.block32 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
            ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb) : "memory");
}
// Instruction descriptor of the 4-bit block-scaled kinds: A and B E2M1 (format 1 of these kinds), both
// K-major, M = 128, N = n, K = 64; E4M3 scales (format 0) per 16 values or E8M0 (format 1) per 32;
// `sf` = the byte of the scale columns this MMA starts at (0, or 2 for the second MMA of a piece).
__host__ __device__ constexpr uint32_t qq_idesc(int n, int vs, uint32_t sf) {
    return (sf << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((vs == 32 ? 1u : 0u) << 23) |
           ((uint32_t)(QQ_BM >> 4) << 24) | (sf << 29);
}
// untiled bulk copy global -> shared, completing on an mbarrier
__device__ __forceinline__ void qq_bulk_load(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// Diagnostic builds only (-DNUVEC_TIMELINE): block (0, 0) records, per role, the clock cycles from the
// kernel's first instruction to the role's start and end, and the cycles inside its waits.
#ifdef NUVEC_TIMELINE
__device__ long long g_qq_timing[3][4];
#define QQT_BEGIN long long qqt_wait_ = 0; const long long qqt_start_ = clock64();
#define QQT_WAIT(...) { const long long qqt_t_ = clock64(); __VA_ARGS__; qqt_wait_ += clock64() - qqt_t_; }
#define QQT_END(role)                                                          \
    if (blockIdx.x == 0 && blockIdx.y == 0) {                                  \
        g_qq_timing[role][0] = qqt_start_ - qqt_entry_;                         \
        g_qq_timing[role][1] = clock64() - qqt_entry_;                          \
        g_qq_timing[role][2] = qqt_wait_;                                       \
    }
#else
#define QQT_BEGIN
#define QQT_WAIT(...) { __VA_ARGS__; }
#define QQT_END(role)
#endif

struct QqParams {
    const uint8_t *sfa, *sfb;  // re-laid-out scales of the weights / the activations
    uint16_t *y;               // bfloat16 [tokens, N]
    int32_t *error;
    int32_t tokens, N, kblocks;
};

template <int BN, int VS>
__global__ void __launch_bounds__(QQ_THREADS, 1)
qqmm_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x, QqParams p) {
#ifdef NUVEC_TIMELINE
    const long long qqt_entry_ = clock64();
#endif
    constexpr uint32_t A_BYTES = QQ_BM * 128, B_BYTES = BN * 128;
    constexpr int PIECES = qq_pieces(VS);                  // scale pieces per 128 rows and stage
    constexpr int STEPS_PER_PIECE = 4 / PIECES;            // MMAs a piece serves: 1 (4 scales per MMA) or 2
    constexpr uint32_t QQ_SF_BYTES = PIECES * 512;
    constexpr uint32_t SFB_BYTES = (BN / 128) * QQ_SF_BYTES;
    constexpr uint32_t STAGE_TX = A_BYTES + B_BYTES + QQ_SF_BYTES + SFB_BYTES;
    // tensor-memory columns behind the accumulator, one set per stage: per piece 4 columns of weight scales
    // (128 rows), then per piece 4 per 128 tokens of activation scales, the tokens' halves side by side
    constexpr int SFB_STEP = 4 * (BN / 128), SFA_COLS = 4 * PIECES, SF_STAGE_COLS = SFA_COLS + SFB_STEP * PIECES;
    constexpr int TMEM_COLS = BN + QQ_STAGES * SF_STAGE_COLS <= 256 ? 256 : 512;
    static_assert(BN + QQ_STAGES * SF_STAGE_COLS <= 512, "accumulator and scale columns exceed tensor memory");
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *as = smem;                                  // [stage][128 rows x 128 B], 128-byte swizzle
    uint8_t *bs = as + QQ_STAGES * A_BYTES;              // [stage][BN rows x 128 B]
    uint8_t *sfa = bs + QQ_STAGES * B_BYTES;             // [stage][pieces x 512 B]
    uint8_t *sfb = sfa + QQ_STAGES * QQ_SF_BYTES;        // [stage][BN / 128][pieces x 512 B]
    uint64_t *bars = reinterpret_cast<uint64_t *>(sfb + QQ_STAGES * SFB_BYTES);
    uint64_t *full = bars, *empty = full + QQ_STAGES, *sfready = empty + QQ_STAGES, *accfull = sfready + QQ_STAGES;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(accfull + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    uint8_t *stage_out = reinterpret_cast<uint8_t *>(bars) + 256;  // epilogue: [4 warps][32 tokens][32 rows] bfloat16

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * QQ_BM, tok0 = blockIdx.y * BN;
    if (tid == 0) {
        for (int s = 0; s < QQ_STAGES; s++) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, 1);
            mbar_init(sfready + s, 4);  // one arrival per epilogue warp
        }
        mbar_init(accfull, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "n"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ── producer: codes by TMA, scales by bulk copies, one barrier per stage ───────────────
        if (lane == 0) {
            asm volatile("griddepcontrol.wait;" ::: "memory");  // the activations' codes and scales are the previous kernel's
            const uint8_t *sfa_src = p.sfa + (size_t)blockIdx.x * p.kblocks * QQ_SF_BYTES;
            const uint8_t *sfb_src = p.sfb + (size_t)blockIdx.y * (BN / 128) * p.kblocks * QQ_SF_BYTES;
            bool ok = true;
            QQT_BEGIN
            for (int kb = 0; kb < p.kblocks && ok; kb++) {
                const uint32_t s = kb % QQ_STAGES, ph = (kb / QQ_STAGES) & 1;
                QQT_WAIT(ok = mbar_wait(empty + s, ph ^ 1, abort_flag))
                if (!ok) break;
                mbar_expect_tx(full + s, STAGE_TX);
                tma_load_2d(as + s * A_BYTES, &tmap_w, kb * 128, n0, full + s);
                tma_load_2d(bs + s * B_BYTES, &tmap_x, kb * 128, tok0, full + s);
                qq_bulk_load(sfa + s * QQ_SF_BYTES, sfa_src + (size_t)kb * QQ_SF_BYTES, QQ_SF_BYTES, full + s);
#pragma unroll
                for (int h = 0; h < BN / 128; h++)
                    qq_bulk_load(sfb + s * SFB_BYTES + h * QQ_SF_BYTES, sfb_src + ((size_t)h * p.kblocks + kb) * QQ_SF_BYTES, QQ_SF_BYTES,
                                 full + s);
            }
            QQT_END(0)
        }
    } else if (warp == 1) {
        // ── MMA issuer: four MMAs of 64 k-values per stage, once the stage's scales are in tensor memory ──
        if (lane == 0) {
            bool ok = true;
            QQT_BEGIN
            for (int kb = 0; kb < p.kblocks && ok; kb++) {
                const uint32_t s = kb % QQ_STAGES, ph = (kb / QQ_STAGES) & 1;
                QQT_WAIT(ok = mbar_wait(full + s, ph, abort_flag) && mbar_wait(sfready + s, ph, abort_flag))
                if (!ok) break;
                tc_fence_after();
                const uint64_t ad = umma_desc(smem_u32(as + s * A_BYTES)), bd = umma_desc(smem_u32(bs + s * B_BYTES));
                const uint32_t sf_cols = tmem_base + BN + s * SF_STAGE_COLS;
#pragma unroll
                for (int step = 0; step < QQ_KB / QQ_STEP; step++) {
                    const int piece = step / STEPS_PER_PIECE;
                    const uint32_t sf = (uint32_t)(step % STEPS_PER_PIECE) * 2u;  // byte of the piece's columns this MMA starts at
                    qq_mma<VS>(tmem_base, ad + (uint64_t)(2 * step), bd + (uint64_t)(2 * step), qq_idesc(BN, VS, sf),
                               (sf_cols + 4 * piece) | (sf << 30), (sf_cols + SFA_COLS + SFB_STEP * piece) | (sf << 30), kb != 0 || step != 0);
                }
                tc_commit(empty + s);
            }
            tc_commit(accfull);
            QQT_END(1)
        }
    } else {
        // ── warps 2-5.  Warp q owns tensor-memory lanes 32 q .. 32 q + 31.  During the main loop it carries
        //    each stage's scales from shared memory to the stage's scale columns of its lanes (every quarter
        //    holds the same columns); then it is the epilogue of weight rows n0 + 32 q + lane. ──
        const int q = warp & 3;
        const uint32_t quarter = tmem_base + ((uint32_t)(q * 32) << 16);
        bool ok = true;
        QQT_BEGIN
        for (int kb = 0; kb < p.kblocks && ok; kb++) {
            const uint32_t s = kb % QQ_STAGES, ph = (kb / QQ_STAGES) & 1;
            // (the stage's columns are free: its data arrived, so the producer saw the MMAs that read them complete)
            QQT_WAIT(ok = mbar_wait(full + s, ph, abort_flag))
            if (!ok) break;
            const uint32_t sf_cols = quarter + BN + s * SF_STAGE_COLS;
#pragma unroll
            for (int piece = 0; piece < PIECES; piece++) {
                qq_st4(sf_cols + 4 * piece, *reinterpret_cast<const uint4 *>(sfa + s * QQ_SF_BYTES + piece * 512 + lane * 16));
#pragma unroll
                for (int h = 0; h < BN / 128; h++)
                    qq_st4(sf_cols + SFA_COLS + SFB_STEP * piece + 4 * h,
                           *reinterpret_cast<const uint4 *>(sfb + s * SFB_BYTES + h * QQ_SF_BYTES + piece * 512 + lane * 16));
            }
            tc_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(sfready + s);
        }
        if (ok) { QQT_WAIT(ok = mbar_wait(accfull, 0, abort_flag)) }
        tc_fence_after();
        const bool wide = (p.N & 7) == 0 && ((uintptr_t)p.y & 15) == 0;
        uint8_t *mine = stage_out + q * 2048;
        const int t8 = lane >> 2, g8 = lane & 3;
#pragma unroll 1
        for (int c = 0; c < BN / 32 && ok; c++) {
            uint32_t v[32];
            tc_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + c * 32, v);
            tc_ld_wait();
            if (tok0 + c * 32 >= p.tokens) continue;
            if (wide) {
#pragma unroll
                for (int j = 0; j < 32; j++)
                    *reinterpret_cast<uint16_t *>(mine + j * 64 + lane * 2) = __bfloat16_as_ushort(__float2bfloat16_rn(__uint_as_float(v[j])));
                __syncwarp();
                const int ng = n0 + q * 32 + g8 * 8;
                uint16_t *dst = p.y + (size_t)(tok0 + c * 32 + t8) * p.N + ng;
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const uint4 piece = *reinterpret_cast<const uint4 *>(mine + (i * 8 + t8) * 64 + g8 * 16);
                    if (ng < p.N && tok0 + c * 32 + i * 8 + t8 < p.tokens) *reinterpret_cast<uint4 *>(dst + (size_t)(i * 8) * p.N) = piece;
                }
                __syncwarp();
            } else {
                const int n = n0 + q * 32 + lane;
                if (n < p.N) {
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const int tok = tok0 + c * 32 + j;
                        if (tok < p.tokens) p.y[(size_t)tok * p.N + n] = __bfloat16_as_ushort(__float2bfloat16_rn(__uint_as_float(v[j])));
                    }
                }
            }
        }
        if (warp == 2 && lane == 0) { QQT_END(2) }
    }
    tc_fence_before();
    __syncthreads();
    if (tid == 0 && *abort_flag && p.error) *p.error = 1;
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "n"(TMEM_COLS) : "memory");
    }
}

typedef CUresult (*QqEncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                               const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                               CUtensorMapFloatOOBfill);

static int32_t qq_map(CUtensorMap *map, const void *base, uint64_t row_bytes, uint64_t rows, uint32_t box_rows) {
    static QqEncodeFn fn = [] {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
            ptr = nullptr;
        return (QqEncodeFn)ptr;
    }();
    if (!fn) return set_error(NVC_ERR_DRIVER, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {row_bytes, rows}, strides[1] = {row_bytes};
    cuuint32_t box[2] = {128, box_rows}, estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error(NVC_ERR_DRIVER, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    return NVC_OK;
}

template <int BN, int VS>
static int32_t qq_launch(nvc_device *dev, const CUtensorMap &mw, const CUtensorMap &mx, const QqParams &p, int64_t tokens, int64_t N) {
    constexpr size_t sf_bytes = qq_pieces(VS) * 512;
    constexpr size_t smem = 1024 + QQ_STAGES * (QQ_BM * 128 + BN * 128 + sf_bytes + (BN / 128) * sf_bytes) + 256 + 4 * 2048;
    auto kernel = qqmm_kernel<BN, VS>;
    static bool configured[64] = {};
    static std::mutex mu;
    if (dev->ordinal < 0 || dev->ordinal >= 64) return set_error(NVC_ERR_UNSUPPORTED, "qqmm: device ordinal %d", dev->ordinal);
    {
        std::lock_guard<std::mutex> g(mu);
        if (!configured[dev->ordinal]) {
            NVC_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            configured[dev->ordinal] = true;
        }
    }
    dim3 grid((unsigned)((N + QQ_BM - 1) / QQ_BM), (unsigned)((tokens + BN - 1) / BN));
    // Programmatic stream serialization: the blocks may start (barriers, tensor memory, descriptors) while the kernel
    // before this one, the activations' quantization, drains; the producer thread synchronises with it on the device
    // (griddepcontrol.wait) before its first load.  NUVEC_PDL=0 restores plain stream order.
    static const bool pdl = [] { const char *e = getenv("NUVEC_PDL"); return !(e && *e == '0'); }();
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(QQ_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = dev->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    NVC_CUDA(cudaLaunchKernelEx(&cfg, kernel, mw, mx, p));
    return check_launch(dev, "qqmm_kernel");
}

}  // namespace nvc

using namespace nvc;

// `prepared`: w_scales already is in the tensor core's layout (nvc_qqmm_prepare_scales).
static int32_t qqmm_impl(nvc_device *dev, const nvc_quant *q, int32_t dtype, const void *x, const uint32_t *w, const void *w_scales, int64_t M,
                         int64_t N, int64_t K, void *y, bool prepared) {
    NVC_TRY(make_current(dev));
    NVC_TRY(check_quant("qqmm", q));
    if (q->mode != NVC_NVFP4 && q->mode != NVC_MXFP4)
        return set_error(NVC_ERR_UNSUPPORTED, "qqmm: nvfp4 and mxfp4 weights take the block-scaled path (mode %d)", q->mode);
    const int vs = q->group_size;  // 16 (nvfp4) or 32 (mxfp4)
    const size_t sf_bytes = (size_t)qq_pieces(vs) * 512;
    if (dtype != NVC_BF16) return set_error(NVC_ERR_UNSUPPORTED, "qqmm: bfloat16 activations only (dtype %d)", dtype);
    if (M < 0 || N < 0 || K < 0 || M > INT32_MAX || N > INT32_MAX || K > INT32_MAX)
        return set_error(NVC_ERR_INVALID_ARGUMENT, "qqmm: invalid shape");
    if (K % QQ_STEP != 0) return set_error(NVC_ERR_UNSUPPORTED, "qqmm: K = %lld is not a multiple of %d", (long long)K, QQ_STEP);
    if (M * N == 0) return NVC_OK;
    if (K == 0) return set_error(NVC_ERR_UNSUPPORTED, "qqmm: empty inner dimension");
    if (!x || !w || !w_scales || !y) return set_error(NVC_ERR_INVALID_ARGUMENT, "qqmm: null operand");
    if ((uintptr_t)w % 16 != 0 || (K / 2) % 16 != 0) return set_error(NVC_ERR_UNSUPPORTED, "qqmm: the packed weights must be 16-byte aligned rows");
    if (dev->capturing) return set_error(NVC_ERR_UNSUPPORTED, "qqmm: not inside a recorded step (it takes scratch from the pool)");

    const int bn = M > 128 ? 256 : 128;
    const int64_t kblocks = (K + QQ_KB - 1) / QQ_KB, wt = (N + 127) / 128, xt = (M + bn - 1) / bn * (bn / 128);
    void *xq = nullptr, *sfa = nullptr, *sfb = nullptr;
    NVC_TRY(dev->pool.alloc((size_t)M * (K / 2), &xq));
    int32_t rc = NVC_OK;
    if (!prepared) rc = dev->pool.alloc((size_t)wt * kblocks * sf_bytes, &sfa);
    if (rc == NVC_OK) rc = dev->pool.alloc((size_t)xt * kblocks * sf_bytes, &sfb);
    auto release = [&]() {  // (the pool hands the blocks out again in stream order)
        if (xq) dev->pool.free(xq);
        if (sfa) dev->pool.free(sfa);
        if (sfb) dev->pool.free(sfb);
    };
    if (rc != NVC_OK) {
        release();
        return rc;
    }
    // x through its quantization: the codes and scales the reference's quantize gives
    // (its scales go straight into the tensor core's layout; rows past M up to the token tile are zero scales)
    const int pieces = qq_pieces(vs);
    rc = quantize_fp4_laid(dev, q, x, M, K, (uint32_t *)xq, (uint8_t *)sfb, kblocks, pieces);
    if (rc == NVC_OK && xt * 128 > (M + 127) / 128 * 128)  // a 256-token tile whose second half holds no rows at all
        rc = cudaMemsetAsync((uint8_t *)sfb + (size_t)((M + 127) / 128) * kblocks * sf_bytes, 0,
                             (size_t)(xt - (M + 127) / 128) * kblocks * sf_bytes, dev->stream) == cudaSuccess
                 ? NVC_OK
                 : set_error(NVC_ERR_DRIVER, "qqmm: cudaMemsetAsync failed");
    if (rc == NVC_OK && !prepared) {
        const int64_t na = wt * kblocks * (int64_t)sf_bytes;
        qq_scale_layout_kernel<<<(unsigned)((na / 16 + 255) / 256), 256, 0, dev->stream>>>((const uint8_t *)w_scales, N, K / vs, (uint8_t *)sfa, wt,
                                                                                           kblocks, pieces);
        rc = check_launch(dev, "qq_scale_layout_kernel");
    }
    CUtensorMap mw, mx;
    if (rc == NVC_OK) rc = qq_map(&mw, w, (uint64_t)K / 2, (uint64_t)N, 128);
    if (rc == NVC_OK) rc = qq_map(&mx, xq, (uint64_t)K / 2, (uint64_t)M, (uint32_t)bn);
    if (rc == NVC_OK) rc = ensure_error_word(dev);
    if (rc == NVC_OK) {
        QqParams p{prepared ? (const uint8_t *)w_scales : (const uint8_t *)sfa, (const uint8_t *)sfb, (uint16_t *)y, dev->error_word_dev, (int32_t)M, (int32_t)N, (int32_t)kblocks};
        if (vs == 16) rc = bn == 256 ? qq_launch<256, 16>(dev, mw, mx, p, M, N) : qq_launch<128, 16>(dev, mw, mx, p, M, N);
        else rc = bn == 256 ? qq_launch<256, 32>(dev, mw, mx, p, M, N) : qq_launch<128, 32>(dev, mw, mx, p, M, N);
    }
    release();
    return rc;
}

extern "C" int32_t nvc_qqmm(nvc_device *dev, const nvc_quant *q, int32_t dtype, const void *x, const uint32_t *w, const void *w_scales, int64_t M,
                            int64_t N, int64_t K, void *y) {
    return qqmm_impl(dev, q, dtype, x, w, w_scales, M, N, K, y, false);
}

extern "C" size_t nvc_qqmm_scales_bytes(const nvc_quant *q, int64_t N, int64_t K) {
    if (!q || (q->group_size != 16 && q->group_size != 32) || N <= 0 || K <= 0) return 0;
    return (size_t)((N + 127) / 128) * (size_t)((K + QQ_KB - 1) / QQ_KB) * (size_t)qq_pieces(q->group_size) * 512;
}

extern "C" int32_t nvc_qqmm_prepare_scales(nvc_device *dev, const nvc_quant *q, const void *w_scales, int64_t N, int64_t K, void *out) {
    NVC_TRY(make_current(dev));
    NVC_TRY(check_quant("qqmm_prepare_scales", q));
    if (q->mode != NVC_NVFP4 && q->mode != NVC_MXFP4) return set_error(NVC_ERR_UNSUPPORTED, "qqmm_prepare_scales: nvfp4 or mxfp4 only");
    if (N < 0 || K < 0 || K % QQ_STEP != 0) return set_error(NVC_ERR_INVALID_ARGUMENT, "qqmm_prepare_scales: invalid shape");
    const size_t bytes = nvc_qqmm_scales_bytes(q, N, K);
    if (bytes == 0) return NVC_OK;
    if (!w_scales || !out || (uintptr_t)out % 16 != 0) return set_error(NVC_ERR_INVALID_ARGUMENT, "qqmm_prepare_scales: null or unaligned operand");
    const int64_t wt = (N + 127) / 128, kblocks = (K + QQ_KB - 1) / QQ_KB;
    qq_scale_layout_kernel<<<(unsigned)((bytes / 16 + 255) / 256), 256, 0, dev->stream>>>((const uint8_t *)w_scales, N, K / q->group_size, (uint8_t *)out, wt,
                                                                                          kblocks, qq_pieces(q->group_size));
    return check_launch(dev, "qq_scale_layout_kernel");
}

extern "C" int32_t nvc_qqmm_prepared(nvc_device *dev, const nvc_quant *q, int32_t dtype, const void *x, const uint32_t *w, const void *laid_out_scales,
                                     int64_t M, int64_t N, int64_t K, void *y) {
    return qqmm_impl(dev, q, dtype, x, w, laid_out_scales, M, N, K, y, true);
}

#ifdef NUVEC_TIMELINE
// Diagnostic build only: out[role][slot] of block (0, 0) in the last qqmm launch; roles 0 producer,
// 1 MMA issuer, 2 warp 2 (scale carrier, then epilogue); slots: cycles from the kernel's entry to the
// role's start, to its end, cycles inside its waits, unused.
extern "C" int32_t nvc_debug_qqmm_timing(long long *out) {
    if (cudaDeviceSynchronize() != cudaSuccess || cudaMemcpyFromSymbol(out, nvc::g_qq_timing, sizeof(long long) * 12) != cudaSuccess)
        return NVC_ERR_DRIVER;
    return NVC_OK;
}
#endif
