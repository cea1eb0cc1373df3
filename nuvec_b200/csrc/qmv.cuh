// Parameter blocks and launch entry points of the few-row product kernels (qmv.cu).
#pragma once
#include "common.cuh"

namespace nvc {

// The ranks' symmetric regions as seen from this device (device memory, read by the kernel).
// Region layout, first bytes: uint32 word `rank` and the word at byte 64 hold the count of fused
// products this rank has finished, the word at byte 68 the blocks of the running kernel that are done.
struct PeerTable {
    void *base[16];
    int32_t rank, size;
};

// Any product the fast kernels do not take.
struct GenericParams {
    int32_t mode, gs, bits, dtype, transpose;
    int32_t scalar_global, expert_global;  // how `global` applies (nvfp4)
    const void *x;
    const uint32_t *w;
    const void *scales, *biases;
    const float *global;
    const uint32_t *lhs, *rhs;  // gathered batches (rhs == nullptr: plain batches)
    uint32_t experts, x_batches;  // what rhs / lhs may address; an index past the end selects the last one
    int64_t M, N, K, ldx, batch;
    int64_t x_batch_stride, w_batch_stride, s_batch_stride;  // elements (w: uint32 words)
    void *y;
};
int32_t launch_generic(nvc_device *dev, const GenericParams &p);

// Fast affine path: bfloat16, transposed weights, up to 8 rows.
struct QmvParams {
    const void *x;
    const uint32_t *w;
    const void *scales, *biases;
    const uint32_t *lhs, *rhs;
    void *y;
    float *partials;     // [tiles][max_parts][128] float32: partial sums of tiles cut by run boundaries
    uint32_t *counters;  // [tiles], zero on entry and on exit
    int64_t N, K, ldx;
    int64_t x_batch_stride, w_batch_stride, s_batch_stride;
    int32_t M, gs, gs_shift, chunk_k, max_parts, x_vec, s_vec;
    uint32_t blk_q, blk_r;  // iterations per block: blk_q, one more in the first blk_r blocks
    // Derived by the launch so that the kernel never divides on its hot paths:
    int32_t row_groups;     // K / group size
    uint32_t row_words;     // K * bits / 32
    int32_t ipt;            // iterations per 16-row tile
    int32_t ci;             // iterations per k-chunk
    int32_t chunk_groups;   // groups per k-chunk
    int32_t tiles;          // 16-row tiles of one product
    int32_t rounds;         // 1: tiles and k-chunks are whole multiples of four iterations
    int32_t xs_pitch;       // words between staged activation rows
    // Gathers: number of weight batches and activation batches the index lists may address; an index
    // past the end selects the last one (the reference's `take` clamps).  0 - 1 = no limit.
    uint32_t experts, x_batches;
    // 1: weights, scales and biases may be read before the previous kernel of the stream has
    // finished (they are constants of the stream's work); 0: nothing is read before it has.
    int32_t early_weights;
    const float *global;       // nvfp4 global scale(s) or nullptr
    int32_t expert_global;     // one value per expert (indexed like the weights' batch)
    // Fused collective (nullptr: plain product).
    const struct PeerTable *peer;
    int32_t peer_rank, peer_size;
    int32_t peer_mode;         // 1: gather of the ranks' [M, N] slices; 2: sum of the ranks' partial [M, N] products into y
    uint64_t peer_out_offset;  // gather: byte offset of the [size, M, N] gathered buffer inside this rank's region
    uint64_t peer_ll_offset;   // byte offset, inside every region, of the two packet areas of size * M * N * 8 bytes
    int32_t *error;            // host-visible word: 2 when the wait for the peers' packets gave up
};
// Returns NVC_ERR_UNSUPPORTED (without setting an error message) when the shape is not one
// the fast kernel takes; the caller then uses the generic kernel.
bool qmv_affine_eligible(int32_t mode, int32_t gs, int32_t bits, int32_t dtype, int32_t transpose, int64_t M,
                         int64_t N, int64_t K, const void *x, int64_t ldx, int64_t x_batch_stride, const uint32_t *w,
                         int64_t w_batch_stride);
// The fast kernel's kind of a (mode, bits) pair: the affine bit width, 40 = mxfp4, 41 = nvfp4, 0 = none.
int qmv_kind(int32_t mode, int32_t bits);
// Caller-provided scratch of fixed capacity (partial sums and arrival counters).
struct QmvScratch {
    float *partials;
    size_t partial_bytes;
    uint32_t *counters;
    size_t counters_len;
};
// `fixed` == nullptr: scratch comes from the device handle's pool and grows on demand.
int32_t launch_qmv_affine(nvc_device *dev, int32_t bits, QmvParams p, int64_t batch, const QmvScratch *fixed = nullptr);

}  // namespace nvc
