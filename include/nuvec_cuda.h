/*
 * nuvec_cuda.h -- C ABI of the B200 (sm_100a) backend for nuvec's quantized-matmul path.
 *
 * The reference (hupe1980/nuvec, Rust) has no C ABI for this path: its evaluator calls GPU
 * back ends through the `GpuEval` seam (crates/nuvec-core/src/gpu.rs:154-281) and its
 * experimental CUDA runtime through Rust crates over the driver API
 * (crates/nuvec-gpu/src/cuda/device.rs:40-227, memory.rs:35-306).  Each entry point below names
 * the reference interface it serves; a Rust `mod cuda` beside `mod metal`/`mod stub` binds
 * these with `extern "C"` and marshals `Primitive::{Quantize, Dequantize, QuantizedMatmul,
 * SortedOffsets}` / `FastOp::GatherQmm` operands to them.
 *
 * Conventions
 *  - Every function returns NVC_OK (0) or a negative nvc_status; the message of the last
 *    failure on the calling thread is read with nvc_last_error().  Nothing aborts or throws
 *    (the reference turns a failed op into a failed array, README.md:102).
 *  - Unless a parameter is documented as a host pointer, every data pointer is a device
 *    pointer, normally from nvc_alloc().  The caller owns inputs and outputs and keeps them
 *    alive until the stream work that uses them has completed.
 *  - All work is enqueued on the device handle's stream and returns without waiting
 *    (the reference's GPU evaluations are asynchronous until `flush`, gpu.rs:1772-1795).
 *  - A handle may be used from any thread, one call at a time per handle.
 *  - dtype codes are nuvec's `DType` discriminants (crates/nuvec-core/src/dtype.rs order, as
 *    used by its fixture files): U8 = 1, U32 = 3, I32 = 7, F16 = 9, BF16 = 10, F32 = 11.
 *  - Empty operands (M == 0, N == 0, no rows) succeed as no-ops
 *    (crates/nuvec-core/tests/quantized.rs:1052-1078).
 */
#ifndef NUVEC_CUDA_H
#define NUVEC_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    NVC_OK = 0,
    NVC_ERR_INVALID_ARGUMENT = -1, /* Error::InvalidArgument, crates/nuvec-core/src/error.rs:17-42 */
    NVC_ERR_UNSUPPORTED = -2,      /* Error::unsupported_dtype / shape the kernels do not take */
    NVC_ERR_OUT_OF_MEMORY = -3,    /* CudaError::OutOfMemory, crates/nuvec-gpu/src/cuda/error.rs:6-42 */
    NVC_ERR_NO_DEVICE = -4,        /* CudaError::NoDevice */
    NVC_ERR_DRIVER = -5,           /* CudaError::Driver{call,message} */
    NVC_ERR_COMM = -6              /* a failed collective (names the call) */
} nvc_status;

enum { NVC_U8 = 1, NVC_U32 = 3, NVC_I32 = 7, NVC_F16 = 9, NVC_BF16 = 10, NVC_F32 = 11 };

/* QuantMode, crates/nuvec-core/src/quantized.rs:24-35 */
enum { NVC_AFFINE = 0, NVC_MXFP4 = 1, NVC_MXFP8 = 2, NVC_NVFP4 = 3 };

/* Quant{mode, group_size, bits}, crates/nuvec-core/src/quantized.rs:94-101.  Checked by every
 * op with the rules of Quant::checked (:137-167): affine group 32/64/128 and bits 1-6 or 8;
 * mxfp4 32/4; mxfp8 32/8; nvfp4 16/4. */
typedef struct {
    int32_t mode;
    int32_t group_size;
    int32_t bits;
} nvc_quant;

typedef struct nvc_device nvc_device; /* opaque: ordinal, stream, pool, scratch */
typedef struct nvc_event nvc_event;   /* opaque: a point on the device's stream */
typedef struct nvc_comm nvc_comm;     /* opaque: one rank of an NCCL communicator */
typedef struct nvc_graph nvc_graph;   /* opaque: a recorded sequence of stream work */

/* DeviceInfo, crates/nuvec-gpu/src/cuda/device.rs:57-75 */
typedef struct {
    char name[128];
    int32_t cc_major, cc_minor;
    int32_t multiprocessors;
    int32_t driver_version;
    uint64_t total_memory;
    uint64_t l2_bytes;
} nvc_info;

/* MemoryStats, crates/nuvec-gpu/src/cuda/memory.rs:16-32 */
typedef struct {
    uint64_t active;  /* bytes handed out and not yet freed */
    uint64_t cached;  /* bytes held by the pool for reuse */
    uint64_t peak;    /* high-water mark of `active` */
    uint64_t limit;   /* allocation limit (default 95% of device memory, memory.rs:64) */
    uint64_t cache_limit;
    uint64_t allocations; /* cudaMalloc calls so far */
} nvc_mem_stats;

/* ── errors ──────────────────────────────────────────────────────────────────────────── */

/* Copies the calling thread's last error message (NUL-terminated) into `buf`. */
void nvc_last_error(char *buf, size_t len);
const char *nvc_version(void);

/* ── device and stream: Device::shared/info/synchronize, device.rs:77-227 ────────────── */

/* Opens device `ordinal` with its own non-blocking stream.  Fails with NVC_ERR_NO_DEVICE when
 * there is no device and NVC_ERR_UNSUPPORTED when it is not compute capability 10.x (the
 * reference refuses devices it has no kernels for, device.rs:107-111). */
int32_t nvc_device_open(int32_t ordinal, nvc_device **out);
int32_t nvc_device_close(nvc_device *dev);
int32_t nvc_device_info(nvc_device *dev, nvc_info *out);
int32_t nvc_synchronize(nvc_device *dev);
/* Adopts an existing cudaStream_t (for example the caller framework's current stream); NULL
 * returns to the handle's own stream.  The previous stream is synchronized first. */
int32_t nvc_device_set_stream(nvc_device *dev, void *cuda_stream);
void *nvc_device_stream(nvc_device *dev);
/* Kernels this handle has launched so far (the reference counts dispatches the same way for
 * its tests, gpu.rs:27). */
uint64_t nvc_launch_count(nvc_device *dev);

/* ── memory: Buffer::new / pool, memory.rs:35-306; Storage, buffer.rs:17-68 ──────────── */

/* Size classes follow memory.rs:54-60 (<= 8 -> 8; < 16 KiB -> next power of two; else whole
 * 16 KiB pages).  Blocks are 256-byte aligned (the reference asks for at least 64,
 * buffer.rs:12-15).  Device memory, not managed memory: host access goes through the copies
 * below. */
int32_t nvc_alloc(nvc_device *dev, size_t bytes, void **out);
int32_t nvc_free(nvc_device *dev, void *ptr);
int32_t nvc_memcpy_h2d(nvc_device *dev, void *dst, const void *host_src, size_t bytes);
int32_t nvc_memcpy_d2h(nvc_device *dev, void *host_dst, const void *src, size_t bytes);
int32_t nvc_memcpy_d2d(nvc_device *dev, void *dst, const void *src, size_t bytes);
int32_t nvc_memset(nvc_device *dev, void *dst, int value, size_t bytes);
/* Pinned host staging memory for the copies above (host pointers). */
int32_t nvc_host_alloc(size_t bytes, void **out);
int32_t nvc_host_free(void *ptr);
int32_t nvc_mem_stats_get(nvc_device *dev, nvc_mem_stats *out);
int32_t nvc_set_memory_limit(nvc_device *dev, uint64_t bytes);
int32_t nvc_set_cache_limit(nvc_device *dev, uint64_t bytes);
int32_t nvc_clear_cache(nvc_device *dev);
int32_t nvc_reset_peak(nvc_device *dev);

/* ── events (timing on the handle's stream; the reference's profiler sums GPU timestamps per
 *    dispatch, crates/nuvec-gpu/src/metal/profile.rs:1-65) ───────────────────────────── */
int32_t nvc_event_create(nvc_device *dev, nvc_event **out);
int32_t nvc_event_destroy(nvc_event *ev);
int32_t nvc_event_record(nvc_device *dev, nvc_event *ev);
int32_t nvc_event_synchronize(nvc_event *ev);
int32_t nvc_event_elapsed_ms(nvc_event *start, nvc_event *stop, float *out_ms);

/* ── recorded command sequences ──────────────────────────────────────────────────────────
 * The reference's evaluator encodes many dispatches into one command buffer and commits it
 * once (`defer` / `commit` / `flush`, crates/nuvec-core/src/gpu.rs:154-281).  The equivalent
 * here: everything enqueued on the handle between begin and end is recorded instead of run,
 * and the recording replays with one launch.  Run the sequence once before recording it, so
 * that scratch buffers exist; allocation, frees and host copies are not allowed while
 * recording. */
int32_t nvc_graph_begin(nvc_device *dev);
int32_t nvc_graph_end(nvc_device *dev, nvc_graph **out);
int32_t nvc_graph_launch(nvc_device *dev, nvc_graph *graph);
int32_t nvc_graph_destroy(nvc_graph *graph);

/* ── the path ────────────────────────────────────────────────────────────────────────── */

/* Primitive::Quantize -> kernels::quantize / fp_quantize
 * (crates/nuvec-core/src/kernels.rs:774-831, 914-971; shape rule primitive.rs:1223-1259).
 * w: [rows, cols] of `dtype` (F16/BF16/F32), cols % group_size == 0.
 * out_codes: uint32 [rows, cols*bits/32].  Affine: out_scales/out_biases [rows, cols/gs] of
 * `dtype`.  Other modes: out_scales uint8, out_biases NULL.  global_scale: one float32 on the
 * device (nvfp4 only) or NULL. */
int32_t nvc_quantize(nvc_device *dev, const nvc_quant *q, int32_t dtype, const void *w,
                     int64_t rows, int64_t cols, const float *global_scale,
                     uint32_t *out_codes, void *out_scales, void *out_biases);

/* Primitive::Dequantize -> kernels::dequantize / fp_dequantize (kernels.rs:835-859, 976-1009).
 * Affine: `dtype` is the dtype of scales, biases and out; `fused` = 0 rounds the product and
 * the sum separately (the reference's CPU result, bit for bit), `fused` = 1 rounds
 * fma(code, scale, bias) once (its Metal kernel, quantized.h:2701-2705).  Other modes: `dtype`
 * is the output dtype, scales are uint8, biases NULL. */
int32_t nvc_dequantize(nvc_device *dev, const nvc_quant *q, int32_t dtype, const uint32_t *codes,
                       const void *scales, const void *biases, const float *global_scale,
                       int64_t rows, int64_t cols, void *out, int32_t fused);

/* FastOp::QuantizeDequantize (crates/nuvec-core/src/products.rs:306-315; MLX's fp_quantize_dequantize): x [rows, cols]
 * through its quantization in a floating-point mode -- the values its codes represent, in x's dtype (with the
 * optional nvfp4 global scale).  The activation side of qqmm and gather_qqmm (products.rs:337-352, 437-463): the
 * reference multiplies the result with nvc_quantized_matmul / nvc_gather_qmm.  Takes scratch from the pool. */
int32_t nvc_quantize_dequantize(nvc_device *dev, const nvc_quant *q, int32_t dtype, const void *x, int64_t rows,
                                int64_t cols, const float *global_scale, void *out);

/* Primitive::QuantizedMatmul (crates/nuvec-core/src/quantized.rs:453-537, shape rule
 * primitive.rs:1279-1323; CPU result kernels.rs:1091-1142).
 *   y[b] = x[b] (M x K, row stride ldx) * dequantize(w[b])^T      (transpose != 0)
 *   y[b] = x[b] (M x K)                 * dequantize(w[b])        (transpose == 0)
 * for b in [0, batch).  w[b] is [N, K*bits/32] (transposed) or [K, N*bits/32]; scales/biases
 * [N, K/gs] or [K, N/gs].  Batch strides are in elements of the operand (0 broadcasts);
 * scales and biases share one batch stride.  `dtype` is the dtype of x, y and (affine) of
 * scales/biases.  y is dense [batch, M, N].  global_scale: one float32 (nvfp4) or NULL. */
int32_t nvc_quantized_matmul(nvc_device *dev, const nvc_quant *q, int32_t dtype,
                             int32_t transpose, const void *x, const uint32_t *w,
                             const void *scales, const void *biases, const float *global_scale,
                             int64_t M, int64_t N, int64_t K, int64_t ldx, int64_t batch,
                             int64_t x_batch_stride, int64_t w_batch_stride,
                             int64_t s_batch_stride, void *y);

/* Primitive::SortedOffsets -> kernels::sorted_offsets (kernels.rs:875-892):
 * out_offsets[g] = number of indices < g, for g in [0, groups); int32. */
int32_t nvc_sorted_offsets(nvc_device *dev, const uint32_t *indices, int64_t rows,
                           int64_t groups, int32_t *out_offsets);

/* FastOp::GatherQmm (crates/nuvec-core/src/quantized.rs:589-719, fast/imp.rs:261-274):
 *   y[i] = x[lhs[i]] (M x K) * dequantize(w[rhs[i]])^T     for i in [0, rows)
 * x: [x_batches, M, K] dense; w: [experts, N, K*bits/32]; scales/biases [experts, N, K/gs];
 * lhs (NULL = 0,1,2,...) and rhs: uint32 [rows]; y: [rows, M, N].  global_scale: float32
 * [experts] (nvfp4) or NULL.  `sorted` != 0 promises rhs is non-decreasing; with M == 1,
 * lhs == NULL and the reference's `grouped(rows, experts)` rule (quantized.rs:724-731) the
 * rows of one expert are multiplied together.  `offsets` (int32 [experts], from
 * nvc_sorted_offsets) may be NULL, in which case it is computed into scratch. */
int32_t nvc_gather_qmm(nvc_device *dev, const nvc_quant *q, int32_t dtype, int32_t transpose,
                       const void *x, const uint32_t *w, const void *scales, const void *biases,
                       const float *global_scale, const uint32_t *lhs, const uint32_t *rhs,
                       const int32_t *offsets, int32_t sorted, int64_t rows, int64_t x_batches,
                       int64_t M, int64_t N, int64_t K, int64_t experts, void *y);

/* qqmm (crates/nuvec-core/src/products.rs:337-352: MLX's qqmm): y = q(x) * w^T with BOTH operands quantized
 * in the weight's mode -- x (bfloat16 [M, K]) goes through its own quantization first (fake_quant, :317-324:
 * the values the codes represent), then the ordinary quantized product.  NVFP4 weights without global
 * scales ([N, K / 8] codes, [N, K / 16] E4M3 scales); K a multiple of 64.  This is the product that the
 * tensor cores' native block-scaled instruction computes (tcgen05.mma.kind::mxf4nvf4.block_scale: both
 * operands as 4-bit codes with their scale factors in tensor memory): within a block of 16 the products and
 * their scaled sum are exact in float32, so only the order of the blocks' addition differs from the
 * reference's float32 product of the dequantized operands.  Takes scratch from the pool (the quantized
 * activations and the two scale arrays in the tensor core's layout): not inside a recorded step. */
int32_t nvc_qqmm(nvc_device *dev, const nvc_quant *q, int32_t dtype, const void *x, const uint32_t *w,
                 const void *w_scales, int64_t M, int64_t N, int64_t K, void *y);
/* The weight's scales laid out once (at load time) the way the tensor core reads them, instead of at every
 * call: nvc_qqmm_scales_bytes gives the size of that array (0 for an unsupported quantization),
 * nvc_qqmm_prepare_scales fills it (out: device memory, 16-byte aligned), nvc_qqmm_prepared is nvc_qqmm with
 * it in place of w_scales. */
size_t nvc_qqmm_scales_bytes(const nvc_quant *q, int64_t N, int64_t K);
int32_t nvc_qqmm_prepare_scales(nvc_device *dev, const nvc_quant *q, const void *w_scales, int64_t N, int64_t K,
                                void *out);
int32_t nvc_qqmm_prepared(nvc_device *dev, const nvc_quant *q, int32_t dtype, const void *x, const uint32_t *w,
                          const void *laid_out_scales, int64_t M, int64_t N, int64_t K, void *y);

/* crate::with_row_exact (crates/nuvec-core/src/lib.rs:160-193): while on, quantized and gathered products of up to
 * 8 rows (ROW_INDEPENDENT_ROWS) give each row the bits of its one-row product: the few-row kernel cuts every such
 * product the way it cuts one row of one batch (the cuts decide the order of a row's float32 sums), rows that do
 * not fit the kernel together run as many at a time as fit, and gathers take the grouped kernel only beyond 64
 * rows (quantized.rs:723-731).  Off by default: products are cut for speed, and a row's bits may depend on the
 * number of rows and batches multiplied with it. */
int32_t nvc_set_row_exact(nvc_device *dev, int32_t on);
int32_t nvc_row_exact(nvc_device *dev);

/* fast::quantized_attention (crates/nuvec-core/src/fast.rs:694-722, fast/imp.rs:3940-4096): attention over an
 * affine-quantized KV cache, without a mask (every query row attends to all S keys; the cache is read once per row),
 *   out[b, h, l, :] = softmax(scale * q[b, h, l, :] . K[b, h / rep, s, :] over s [, sinks[h]]) . V[b, h / rep, s, :]
 * q and out [B, Hq, L, D] of `dtype` (float16 / bfloat16 / float32), K and V codes uint32 [B, Hkv, S, D * bits / 32],
 * their scales and biases [B, Hkv, S, D / group_size] of `dtype`, sinks [Hq] of `dtype` or NULL (a sink joins the
 * softmax's denominator only).  `capacity` >= S is the number of rows between consecutive heads of every cache
 * tensor (a cache is a view of a longer allocation).  The shapes the reference's kernel takes: D 64 or 128; 3, 4 or
 * 8 bits; groups of 32, 64 or 128 within a head; Hq / Hkv 1, 2, 4 or 8.  Float32 throughout: within the float bound
 * of attention over the dequantized cache (crates/nuvec-core/tests/quantized.rs:1964-2031).  The splits' partial
 * results use the handle's scratch block: inside a recorded step only shapes whose scratch (B * Hq * splits *
 * (D + 2) floats, at most a few MB) the handle already holds -- run the shape once before recording.  `causal` != 0: query row l stands at position S - L + l and attends to the keys
 * up to it (AttentionMask::Causal over a cache that already holds the L new keys, crates/nuvec-lm/src/model.rs:1293-1340). */
int32_t nvc_quantized_attention(nvc_device *dev, const nvc_quant *quant, int32_t dtype, const void *q,
                                const uint32_t *k_codes, const void *k_scales, const void *k_biases,
                                const uint32_t *v_codes, const void *v_scales, const void *v_biases, const void *sinks,
                                int64_t B, int64_t Hq, int64_t Hkv, int64_t L, int64_t S, int64_t D, int64_t capacity,
                                float scale, int32_t causal, void *out);

/* convert_packed (crates/nuvec-lm/src/quant.rs:36-199) for one layer of an AutoAWQ or GPTQ checkpoint, on the
 * device: qweight (int32, AWQ [inputs, outputs / 8], GPTQ [inputs * bits / 32, outputs]), qzeros (int32
 * [groups, outputs * bits / 32], or NULL for the symmetric zero 2^(bits - 1); GPTQ v1 stores zero - 1) and
 * scales ([groups, outputs], float16 / bfloat16 / float32) become MLX's affine layout: codes uint32
 * [outputs, inputs * bits / 32], scales and biases [outputs, groups] with bias = -zero * scale (float32
 * product, rounded to the scales' type).  bits 2, 4 or 8 (AWQ: 4); inputs a multiple of group_size.  GPTQ's
 * g_idx is the caller's to check (it must be the identity grouping, quant.rs:97-111). */
enum { NVC_PACKED_AWQ = 0, NVC_PACKED_GPTQ_V1 = 1, NVC_PACKED_GPTQ_V2 = 2 };
int32_t nvc_convert_packed(nvc_device *dev, int32_t format, int32_t bits, int32_t group_size, int32_t scale_dtype,
                           const int32_t *qweight, const int32_t *qzeros, const void *scales, int64_t inputs,
                           int64_t outputs, uint32_t *out_codes, void *out_scales, void *out_biases);

/* `v[..., first::step, :]` of a dense array seen as [outer, n, inner_bytes]: out[o, j, :] = src[o, first + j * step, :]
 * for j < ceil((n - first) / step).  With step 2 it takes apart the interleaved gate and up rows of gpt-oss's
 * fused experts (`v.take(arange(first, n, 2), axis)`, crates/nuvec-lm/src/lib.rs:414-420, 431-440). */
int32_t nvc_take_strided(nvc_device *dev, const void *src, int64_t outer, int64_t n, int64_t inner_bytes,
                         int64_t first, int64_t step, void *out);

/* fast::moe_route (crates/nuvec-core/src/fast/imp.rs:2652-2672; kernel crates/nuvec-kernels/src/metal/moe.metal):
 * per row of `experts` router probabilities (float dtype, dense [rows, experts]) the indices
 * (uint32 [rows, k]) of the k largest in the stable ascending order of a sort with NaN last, and
 * those probabilities ([rows, k], same dtype), divided by their sum when `normalize` is set.  At
 * most 1024 experts.  The results are the bits of the reference's CPU composition
 * (argpartition, take_along_axis, sum, divide). */
int32_t nvc_moe_route(nvc_device *dev, int32_t dtype, const void *probs, int64_t rows, int64_t experts,
                      int64_t k, int32_t normalize, uint32_t *out_indices, void *out_scores);
/* fast::weighted_sum (fast/imp.rs:2731-2747): out[r, :] = sum over j of x[r, j, :] * w[r, j] for
 * x [rows, k, d] and w [rows, k] of one float dtype; products rounded to the dtype, the sum taken in
 * float64 in order and rounded once, as the reference's CPU composition does. */
int32_t nvc_weighted_sum(nvc_device *dev, int32_t dtype, const void *x, const void *w, int64_t rows,
                         int64_t k, int64_t d, void *out);
/* The bias of SwitchProjection::forward (crates/nuvec-lm/src/model.rs:2139-2143: `y.add(bias.take(indices, 0))`
 * after gather_qmm): y[r, :] += bias[indices[r], :] in place, for y [rows, n] and bias [experts, n] of one
 * float dtype and uint32 indices [rows]; float32 arithmetic and one rounding for the halves; an index past
 * the end takes the last expert's bias, as `take` clamps (crates/nuvec-core/src/kernels.rs:120-133). */
int32_t nvc_expert_bias_add(nvc_device *dev, int32_t dtype, void *y, const void *bias, const uint32_t *indices,
                            int64_t rows, int64_t n, int64_t experts);

/* The bookkeeping of SwitchGlu::forward for many rows (crates/nuvec-lm/src/model.rs:2199-2210), all uint32 [pairs]:
 *   out_order    the stable ascending argsort of the flattened expert indices (pairs = tokens x k;
 *                crates/nuvec-core/src/kernels.rs:231-266),
 *   out_restore  its inverse (the argsort of out_order): where each pair went,
 *   out_tokens   each sorted pair's token, out_order / k (may be NULL),
 *   out_sorted   each sorted pair's expert (may be NULL),
 *   out_offsets  int32 [experts]: the experts' first rows, what nvc_sorted_offsets gives for out_sorted (may be NULL).
 * Indices must be smaller than `experts` (at most 1024). */
int32_t nvc_moe_sort(nvc_device *dev, const uint32_t *indices, int64_t pairs, int64_t k, int64_t experts,
                     uint32_t *out_order, uint32_t *out_restore, uint32_t *out_tokens, uint32_t *out_sorted,
                     int32_t *out_offsets);
/* take(src, indices, 0) of whole rows (the activations by token before the experts, the results back into
 * pair order after them): out[i, :] = src[indices[i], :] for rows of row_bytes bytes; an index past the
 * end takes the last row (kernels.rs:120-133). */
int32_t nvc_take_rows(nvc_device *dev, const void *src, int64_t src_rows, int64_t row_bytes, const uint32_t *indices,
                      int64_t n, void *out);
/* fast::rms_norm and fast::add_rms_norm (crates/nuvec-core/src/fast/imp.rs:358-412), the normalisation in front
 * of a layer's projections: y[r, :] = x[r, :] / sqrt(mean(x[r, :]^2) + eps) * weight over rows of d elements
 * of one float dtype (weight [d] or NULL); add_rms_norm first stores out_sum = x + residual (rounded to the
 * dtype) and normalises that.  The arithmetic is the CPU expansion's (fast/imp.rs:1367-1379): float32 squares,
 * their sum in float64 over 8 lanes combined by a fixed tree (kernels.rs:611-624) and rounded to float32,
 * times float32(1 / d), plus eps, 1 / sqrt, x times that rounded to the dtype, times the weight rounded
 * again -- every step an IEEE operation in the reference's order, so the results are its bits. */
int32_t nvc_rms_norm(nvc_device *dev, int32_t dtype, const void *x, const void *weight, float eps, int64_t rows,
                     int64_t d, void *y);
int32_t nvc_add_rms_norm(nvc_device *dev, int32_t dtype, const void *x, const void *residual, const void *weight,
                         float eps, int64_t rows, int64_t d, void *out_sum, void *y);
/* QuantizedEmbedding::forward (crates/nuvec-nn/src/layers.rs:246-255): the rows of a quantized table
 * (codes [vocab, cols * bits / 32], scales and biases [vocab, cols / group_size]) picked by uint32 ids
 * [count] and dequantized with nvc_dequantize's arithmetic into out [count, cols] of `dtype` (the scales'
 * dtype for affine tables); an id past the end takes the last row, as `take` clamps
 * (crates/nuvec-core/src/kernels.rs:120-133). */
int32_t nvc_quantized_embedding(nvc_device *dev, const nvc_quant *q, int32_t dtype, const uint32_t *codes,
                                const void *scales, const void *biases, int64_t vocab, int64_t cols,
                                const uint32_t *ids, int64_t count, void *out);
/* The activation between the up / gate and the down products (SwitchGlu::through,
 * crates/nuvec-lm/src/model.rs:2160-2171): nuvec_nn::swiglu = silu(gate) * up and gpt-oss's clamped
 * nuvec_nn::swiglu_oai = (clip(up, -limit, limit) + 1) * g * sigmoid(alpha * g) with g = min(gate, limit)
 * (crates/nuvec-nn/src/lib.rs:513-579), over n elements of one float dtype.  The arithmetic is the reference's
 * CPU evaluation of the compiled function -- its operations one by one, each rounded to the dtype
 * (crates/nuvec-core/src/fused.rs:214-217), MLX's sigmoid in float32 (kernels.rs:1538-1543), alpha and limit
 * rounded to the dtype first.  The exponential is the one step that is not an IEEE operation: where the
 * device's and the host's differ in their last bit, a result can differ by a unit or two in the last place. */
int32_t nvc_swiglu(nvc_device *dev, int32_t dtype, const void *gate, const void *up, int64_t n, void *out);
int32_t nvc_swiglu_oai(nvc_device *dev, int32_t dtype, const void *gate, const void *up, float alpha, float limit,
                       int64_t n, void *out);

/* The same product with HOST operands for the activations and the result: copies x in,
 * multiplies, copies y out and waits.  This is what an evaluator whose arrays live in host
 * memory calls per step (the reference's CPU arrays, buffer.rs:17-27); the weights stay
 * resident on the device. */
int32_t nvc_quantized_matmul_host(nvc_device *dev, const nvc_quant *q, int32_t dtype,
                                  int32_t transpose, const void *host_x, const uint32_t *w,
                                  const void *scales, const void *biases,
                                  const float *global_scale, int64_t M, int64_t N, int64_t K,
                                  void *host_y);

/* The asynchronous form: returns as soon as the copies and the kernel are on the stream.  The
 * result is PENDING, as a GPU result is in the reference's evaluator until `flush`
 * (crates/nuvec-core/src/gpu.rs:1772-1795): nvc_synchronize (or any call that synchronizes, e.g.
 * nvc_memcpy_d2h) delivers it into host_y.  host_x may be reused when the call returns; host_y must
 * stay valid until the synchronization.  A decode step issues its products back to back and waits once. */
int32_t nvc_quantized_matmul_host_async(nvc_device *dev, const nvc_quant *q, int32_t dtype,
                                        int32_t transpose, const void *host_x, const uint32_t *w,
                                        const void *scales, const void *biases,
                                        const float *global_scale, int64_t M, int64_t N, int64_t K,
                                        void *host_y);

/* A list of such products in one call (an evaluator walking the nodes of a step between two
 * flushes); the fields are the arguments of nvc_quantized_matmul_host_async.  All activations travel
 * in one copy.  A list that arrives again unchanged after a synchronization (the same weights, sizes
 * and host buffers: a decode loop) is recorded the second time and replayed from then on, so the
 * step costs one copy and one graph launch; the contents of the host buffers are read anew at every
 * call.  Any other list drops the recording. */
typedef struct {
    nvc_quant quant;
    int32_t dtype, transpose;
    const void *host_x;
    const uint32_t *w;
    const void *scales, *biases;
    const float *global_scale;
    int64_t M, N, K;
    void *host_y;
} nvc_host_product;
int32_t nvc_quantized_matmul_host_batch(nvc_device *dev, const nvc_host_product *items, size_t count);

/* No counterpart in the reference.  The few-row product for callers that may not allocate device
 * memory while they run: code that executes between a memory reservation made up front and its
 * release (a serving loop under a fixed memory budget, a plugin hosted by a runtime that owns
 * the allocator), where a hidden cudaMalloc would either fail or break the budget.  The other
 * entry points take their scratch (partial sums of tiles split across warps, arrival counters)
 * from the handle's pool and may grow it; this one keeps that scratch in a 4 MiB array that is
 * part of the library image -- every GPU that loads the library holds it until the process
 * exits -- and calls no cudaMalloc, cudaFree or allocating routine.
 *   x: bfloat16 [M, K] dense, 1 <= M <= 8;  w: affine 2-, 3-, 4-, 6- or 8-bit, [N, K*bits/32], K a multiple
 *   of 32 values per vector-load step (any K the fast kernel of nvc_quantized_matmul takes);
 *   scales/biases bfloat16 [N, K/gs];  y: bfloat16 [M, N].  Results equal nvc_quantized_matmul's.
 * Limit: the partial sums of tiles that block boundaries cut (one slot per block of the launch, each
 * of as many 512-byte partial tiles as a tile can be cut into) must fit 4 MiB - 64 KiB: every decode
 * projection does, by three orders of magnitude; a product of few rows and a very long K spread over
 * all multiprocessors (say N = 304, K = 65536) does not and gets NVC_ERR_UNSUPPORTED with the sizes
 * in the message.  The first call on a device looks up the array's device address; make that
 * call before any stream capture.  All calls share the one array: it keeps the last call's
 * contents (the counters are cleared on the stream at the start of each call), and two calls
 * whose kernels overlap on the GPU -- different streams, different handles -- race on it. */
int32_t nvc_quantized_matmul_noalloc(nvc_device *dev, const nvc_quant *q, const void *x, const uint32_t *w,
                                     const void *scales, const void *biases, int64_t M, int64_t N, int64_t K,
                                     void *y);

/* ── collectives: trait Communicator, crates/nuvec-core/src/distributed.rs:43-83 ────── */

/* One rank per process and per GPU (distributed.rs:145-180).  The 128-byte id is created on
 * rank 0 and carried to the other ranks by the caller's bootstrap (the reference uses a
 * hostfile, crates/nuvec-distributed/src/backend.rs:79-100). */
int32_t nvc_comm_unique_id(uint8_t out_id[128]);
int32_t nvc_comm_init(nvc_device *dev, int32_t rank, int32_t size, const uint8_t id[128],
                      nvc_comm **out);
/* The same with a host-side time limit (milliseconds; 0 = the default): a rank that never joins
 * ends the call with NVC_ERR_COMM after the limit instead of blocking for ever, and the
 * half-built communicator is aborted.  nvc_comm_init uses NUVEC_DISTRIBUTED_TIMEOUT seconds (the
 * reference's variable, crates/nuvec-distributed/src/backend.rs:44-59), 120 when it is unset. */
int32_t nvc_comm_init_timeout(nvc_device *dev, int32_t rank, int32_t size, const uint8_t id[128],
                              int64_t timeout_ms, nvc_comm **out);
int32_t nvc_comm_rank(nvc_comm *comm);
int32_t nvc_comm_size(nvc_comm *comm);
/* Communicator::all_gather(&[u8], &mut [u8]) (distributed.rs:52; ring.rs:868-889): recv holds
 * size * bytes_per_rank bytes, rank r's block at offset r * bytes_per_rank.  In place when
 * send == recv + rank * bytes_per_rank. */
int32_t nvc_all_gather(nvc_comm *comm, const void *send, void *recv, size_t bytes_per_rank);
/* Communicator::all_reduce(op, dtype, &mut [u8]) (distributed.rs:50), in place; op is one of
 * AllReduce::{Sum, Max, Min} (distributed.rs:32-39). */
#define NVC_REDUCE_SUM 0
#define NVC_REDUCE_MAX 1
#define NVC_REDUCE_MIN 2
int32_t nvc_all_reduce(nvc_comm *comm, int32_t op, int32_t dtype, void *buf, size_t count);
int32_t nvc_all_reduce_sum(nvc_comm *comm, int32_t dtype, void *buf, size_t count);
/* Communicator::send / recv (distributed.rs:54-57): `bytes` bytes to / from rank `peer`, ordered on
 * the device's stream; a send pairs with the peer's recv of the same size. */
int32_t nvc_send(nvc_comm *comm, const void *buf, size_t bytes, int32_t peer);
int32_t nvc_recv(nvc_comm *comm, void *buf, size_t bytes, int32_t peer);
/* Communicator::health (distributed.rs:66-70): NVC_OK or NVC_ERR_COMM with the async error. */
int32_t nvc_comm_health(nvc_comm *comm);
int32_t nvc_comm_abort(nvc_comm *comm);
int32_t nvc_comm_destroy(nvc_comm *comm);

/* ── sharded few-row products fused with their collective ──────────────────────────────────
 *
 * Replace the pairs "quantized_matmul on this rank's rows of W, then Communicator::all_gather"
 * (crates/nuvec-core/src/distributed.rs:52, 695-700; the sharded logits of
 * crates/nuvec-lm/src/model.rs:3336-3346) and "quantized_matmul on this rank's columns of W, then
 * all_sum" (ShardedToAllLinear::forward, crates/nuvec-nn/src/sharded.rs:195-202) for few-row products.
 * The product kernel itself sends every result to the other ranks over NVLink peer stores as
 * 8-byte packets {value, sequence number}; at its end the same kernel collects the packets the other
 * ranks sent to this one (a reader that sees the product's sequence number has the value with it:
 * no fence, no flag, no collective library).  When the kernel ends the result is complete on this
 * rank, so the next kernel of the stream needs no wait of its own.
 *
 * Set-up, once: every rank allocates a symmetric region of the same size (nvc_symm_alloc), the
 * caller's bootstrap carries the 64-byte handles to the other ranks, every rank opens the others'
 * regions (nvc_symm_open) and builds a group from the table of base addresses (its own included,
 * at index `rank`).  A region starts zeroed; its first 4 KiB belong to the group (sequence
 * counters), the products' buffers live behind NVC_SYMM_RESERVED at offsets that are multiples of
 * 256 and the same on every rank.
 *
 * Rules: every rank of the group issues the same sequence of fused products.  A product's buffers
 * inside the regions (its footprint) may be reused by a later product; the packet areas alternate
 * between two halves, so a rank that runs ahead by one product never lands on packets still being
 * read, and it cannot run ahead by two (it needs the slower rank's packets of the product between).
 * Only this rank's own kernel writes this rank's gathered buffer (the other ranks write packets,
 * never results), so reading a gathered buffer as the activations of a later product is safe in
 * stream order.  A wait that gives up (about a second) sets the device's error word:
 * nvc_synchronize reports it, and the device stays usable. */
#define NVC_SYMM_RESERVED 4096
typedef struct { uint8_t bytes[64]; } nvc_ipc_handle;
typedef struct nvc_peer_group nvc_peer_group; /* opaque: the ranks' region addresses on this device */

int32_t nvc_symm_alloc(nvc_device *dev, size_t bytes, void **out_ptr, nvc_ipc_handle *out_handle);
int32_t nvc_symm_open(nvc_device *dev, const nvc_ipc_handle *handle, void **out_peer_ptr);
int32_t nvc_symm_close(nvc_device *dev, void *peer_ptr);
int32_t nvc_symm_free(nvc_device *dev, void *ptr);
/* region_bytes: the size every rank allocated; products whose footprint would pass it are refused. */
int32_t nvc_peer_group_create(nvc_device *dev, int32_t rank, int32_t size, void *const *region_bases,
                              size_t region_bytes, nvc_peer_group **out);
int32_t nvc_peer_group_destroy(nvc_peer_group *group);
/* Bytes a fused product occupies in every region from its offset on (a multiple of 256): the
 * gathered [size, M, N_local] bfloat16 buffer followed by the packet areas / the packet areas alone. */
size_t nvc_gather_footprint(int32_t size, int64_t M, int64_t N_local);
size_t nvc_all_sum_footprint(int32_t size, int64_t M, int64_t N);
/* N-sharded product + all_gather.  This rank multiplies its rows of W (w, scales, biases: [N_local, ..]);
 * the gathered result, bfloat16 [size, M, N_local] (rank r's slice at index r: the layout of
 * all_gather along axis 0), ends up at byte offset out_offset of THIS rank's region on every rank.
 * Operands as nvc_quantized_matmul_noalloc (bfloat16, affine 2/3/4/6/8 bits, M <= 8). */
int32_t nvc_quantized_matmul_gather(nvc_device *dev, nvc_peer_group *group, const nvc_quant *q, const void *x,
                                    const uint32_t *w, const void *scales, const void *biases, int64_t M,
                                    int64_t N_local, int64_t K, size_t out_offset);
/* K-sharded product + all_sum.  This rank multiplies its K_local columns of W (w: [N, K_local * bits / 32],
 * scales / biases: [N, K_local / group_size]) by its K_local columns of the activations (x: [M, K_local]);
 * y (device memory, bfloat16 [M, N]) receives the sum of all ranks' float32 partial products, added in
 * rank order and rounded once, bit-identical on every rank.  The packet areas occupy
 * nvc_all_sum_footprint bytes at scratch_offset of every region. */
int32_t nvc_quantized_matmul_all_sum(nvc_device *dev, nvc_peer_group *group, const nvc_quant *q, const void *x,
                                     const uint32_t *w, const void *scales, const void *biases, int64_t M,
                                     int64_t N, int64_t K_local, void *y, size_t scratch_offset);

#ifdef __cplusplus
}
#endif
#endif /* NUVEC_CUDA_H */
