// Entry points of the product operations: argument checks with the reference's rules and
// messages (crates/nuvec-core/src/quantized.rs:137-167, 363-379, 453-537, 589-673;
// crates/nuvec-core/src/primitive.rs:1279-1323) and the choice of kernel, which plays the part
// of the reference's Metal routing (crates/nuvec-core/src/gpu.rs:6934-7168, 7174-7294):
// few rows -> qmv, many rows -> qmm on tcgen05, anything else -> the generic kernel.
#include "qmm.cuh"
#include "qmv.cuh"

#include <cstdlib>
#include <cstring>

namespace nvc {

static int32_t check_product(const char *op, const nvc_quant *q, int32_t dtype, int32_t transpose, const void *biases,
                             const float *global, int64_t M, int64_t N, int64_t K) {
    NVC_TRY(check_quant(op, q));
    if (!is_float_dtype(dtype)) return set_error(NVC_ERR_UNSUPPORTED, "%s: unsupported dtype %d", op, dtype);
    if (q->mode == NVC_AFFINE && !biases)
        return set_error(NVC_ERR_INVALID_ARGUMENT, "%s: biases must be provided for affine quantization", op);
    if (q->mode != NVC_AFFINE && biases)
        return set_error(NVC_ERR_INVALID_ARGUMENT, "%s: biases must be null for this quantization mode", op);
    if (global && q->mode != NVC_NVFP4)
        return set_error(NVC_ERR_INVALID_ARGUMENT, "%s: a global scale is only supported for nvfp4", op);
    if (M < 0 || N < 0 || K < 0) return set_error(NVC_ERR_INVALID_ARGUMENT, "%s: negative dimension", op);
    int64_t cols = transpose ? K : N;
    if (cols % q->group_size != 0)
        return set_error(NVC_ERR_INVALID_ARGUMENT, "%s: %lld columns are not divisible by the group size %d", op,
                         (long long)cols, q->group_size);
    return NVC_OK;
}

// The reference's rule for the grouped kernel (quantized.rs:724-731): at least 16 rows and 4
// per expert on average.
// Row-exact (crate::with_row_exact): more rows than the row-independent region, 8 tokens with up to 8 experts.
static bool grouped(int64_t rows, int64_t experts, bool row_exact) {
    return rows >= (row_exact ? 65 : 16) && rows / (experts > 0 ? experts : 1) >= 4;
}

extern "C" int32_t nvc_set_row_exact(nvc_device *dev, int32_t on) {
    if (!dev) return set_error(NVC_ERR_INVALID_ARGUMENT, "set_row_exact: null device");
    dev->row_exact = on != 0;
    return NVC_OK;
}
extern "C" int32_t nvc_row_exact(nvc_device *dev) { return dev && dev->row_exact ? 1 : 0; }

__global__ void sorted_offsets_kernel(const uint32_t *__restrict__ idx, int64_t rows, int64_t groups,
                                      int32_t *__restrict__ out) {
    int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (g >= groups) return;
    int64_t lo = 0, hi = rows;  // first index whose value is not below g
    while (lo < hi) {
        int64_t mid = lo + (hi - lo) / 2;
        if ((int64_t)idx[mid] < g) lo = mid + 1;
        else hi = mid;
    }
    out[g] = (int32_t)lo;
}

static int32_t run_sorted_offsets(nvc_device *dev, const uint32_t *indices, int64_t rows, int64_t groups,
                                  int32_t *out) {
    if (groups == 0) return NVC_OK;
    sorted_offsets_kernel<<<(unsigned)((groups + 127) / 128), 128, 0, dev->stream>>>(indices, rows, groups, out);
    return check_launch(dev, "sorted_offsets_kernel");
}

}  // namespace nvc

using namespace nvc;

extern "C" int32_t nvc_sorted_offsets(nvc_device *dev, const uint32_t *indices, int64_t rows, int64_t groups,
                                      int32_t *out_offsets) {
    NVC_TRY(make_current(dev));
    if (rows < 0 || groups < 0) return set_error(NVC_ERR_INVALID_ARGUMENT, "sorted_offsets: negative size");
    if (groups > 0 && !out_offsets) return set_error(NVC_ERR_INVALID_ARGUMENT, "sorted_offsets: null output");
    if (rows > 0 && !indices) return set_error(NVC_ERR_INVALID_ARGUMENT, "sorted_offsets: null indices");
    return run_sorted_offsets(dev, indices, rows, groups, out_offsets);
}

extern "C" int32_t nvc_quantized_matmul(nvc_device *dev, const nvc_quant *q, int32_t dtype, int32_t transpose,
                                        const void *x, const uint32_t *w, const void *scales, const void *biases,
                                        const float *global_scale, int64_t M, int64_t N, int64_t K, int64_t ldx,
                                        int64_t batch, int64_t x_batch_stride, int64_t w_batch_stride,
                                        int64_t s_batch_stride, void *y) {
    NVC_TRY(make_current(dev));
    NVC_TRY(check_product("quantized_matmul", q, dtype, transpose, biases, global_scale, M, N, K));
    if (batch < 0 || ldx < K || x_batch_stride < 0 || w_batch_stride < 0 || s_batch_stride < 0)
        return set_error(NVC_ERR_INVALID_ARGUMENT, "quantized_matmul: invalid strides (ldx %lld, K %lld)", (long long)ldx,
                         (long long)K);
    if (batch == 0 || M == 0 || N == 0) return NVC_OK;
    if (!x || !w || !scales || !y) return set_error(NVC_ERR_INVALID_ARGUMENT, "quantized_matmul: null operand");
    if (K == 0) {
        NVC_CUDA(cudaMemsetAsync(y, 0, (size_t)(batch * M * N) * dtype_size(dtype), dev->stream));
        return NVC_OK;
    }
    if (M <= 8 && qmv_affine_eligible(q->mode, q->group_size, q->bits, dtype, transpose, M, N, K, x, ldx,
                                      x_batch_stride, w, w_batch_stride)) {
        QmvParams p{};
        p.x = x; p.w = w; p.scales = scales; p.biases = biases; p.lhs = nullptr; p.rhs = nullptr; p.y = y;
        p.N = N; p.K = K; p.ldx = ldx;
        p.x_batch_stride = x_batch_stride; p.w_batch_stride = w_batch_stride; p.s_batch_stride = s_batch_stride;
        p.M = (int32_t)M; p.gs = q->group_size;
        p.x_vec = ((uintptr_t)x % 16 == 0) && (ldx % 8 == 0) && (x_batch_stride % 8 == 0);
        p.global = global_scale; p.expert_global = 0;
        return launch_qmv_affine(dev, qmv_kind(q->mode, q->bits), p, batch);
    }
    if (dev->row_exact && M > 1 && M <= 8 &&
        qmv_affine_eligible(q->mode, q->group_size, q->bits, dtype, transpose, 1, N, K, x, ldx, x_batch_stride, w, w_batch_stride)) {
        // Row-exact and too many rows for the few-row kernel's shared memory at once: as many rows at a time as fit
        // (every launch is cut like a one-row product, so every row keeps its one-row bits).
        int64_t fit = 1;
        while (fit + 1 <= M && qmv_affine_eligible(q->mode, q->group_size, q->bits, dtype, transpose, fit + 1, N, K, x, ldx, x_batch_stride, w,
                                                   w_batch_stride))
            fit++;
        const size_t esz = dtype_size(dtype);
        for (int64_t r0 = 0; r0 < M; r0 += fit) {
            const int64_t m = M - r0 < fit ? M - r0 : fit;
            for (int64_t b = 0; b < batch; b++) {
                QmvParams p{};
                p.x = (const char *)x + (b * x_batch_stride + r0 * ldx) * esz;
                p.w = w + b * w_batch_stride;
                const size_t ssz = q->mode == NVC_AFFINE ? esz : 1;
                p.scales = (const char *)scales + b * s_batch_stride * ssz;
                p.biases = biases ? (const char *)biases + b * s_batch_stride * ssz : nullptr;
                p.lhs = nullptr; p.rhs = nullptr;
                p.y = (char *)y + (b * M + r0) * N * esz;
                p.N = N; p.K = K; p.ldx = ldx;
                p.x_batch_stride = 0; p.w_batch_stride = 0; p.s_batch_stride = 0;
                p.M = (int32_t)m; p.gs = q->group_size;
                p.x_vec = ((uintptr_t)p.x % 16 == 0) && (ldx % 8 == 0);
                p.global = global_scale; p.expert_global = 0;
                NVC_TRY(launch_qmv_affine(dev, qmv_kind(q->mode, q->bits), p, 1));
            }
        }
        return NVC_OK;
    }
    if (qmm_eligible(q->mode, q->group_size, q->bits, dtype, transpose, M, N, K, x, ldx, w)) {
        for (int64_t b = 0; b < batch; b++) {
            QmmParams p{};
            p.mode = q->mode; p.gs = q->group_size; p.bits = q->bits;
            p.x = (const char *)x + b * x_batch_stride * dtype_size(dtype);
            p.w = w + b * w_batch_stride;
            size_t ssz = q->mode == NVC_AFFINE ? dtype_size(dtype) : 1;
            p.scales = (const char *)scales + b * s_batch_stride * ssz;
            p.biases = biases ? (const char *)biases + b * s_batch_stride * ssz : nullptr;
            p.global = global_scale; p.expert_global = 0; p.offsets = nullptr; p.experts = 1;
            p.rows = M; p.N = N; p.K = K; p.ldx = ldx;
            p.y = (char *)y + b * M * N * dtype_size(dtype);
            NVC_TRY(launch_qmm(dev, p));
        }
        return NVC_OK;
    }
    // Many rows of a bit width only the few-row kernel decodes fast (3 and 6 bits): eight rows at a
    // time through it.  The weights are streamed once per eight rows (from L2 when they fit), which
    // is far from the tensor-core kernel but two orders of magnitude ahead of the generic one.
    if (M > 8 && q->mode == NVC_AFFINE &&
        qmv_affine_eligible(q->mode, q->group_size, q->bits, dtype, transpose, 8, N, K, x, ldx, 0, w, 0)) {
        const size_t esz = dtype_size(dtype);
        for (int64_t b = 0; b < batch; b++) {
            for (int64_t r0 = 0; r0 < M; r0 += 8) {
                const int64_t m = M - r0 < 8 ? M - r0 : 8;
                QmvParams p{};
                p.x = (const char *)x + (b * x_batch_stride + r0 * ldx) * esz;
                p.w = w + b * w_batch_stride;
                p.scales = (const char *)scales + b * s_batch_stride * esz;
                p.biases = (const char *)biases + b * s_batch_stride * esz;
                p.lhs = nullptr; p.rhs = nullptr;
                p.y = (char *)y + (b * M + r0) * N * esz;
                p.N = N; p.K = K; p.ldx = ldx;
                p.x_batch_stride = 0; p.w_batch_stride = 0; p.s_batch_stride = 0;
                p.M = (int32_t)m; p.gs = q->group_size;
                p.x_vec = ((uintptr_t)p.x % 16 == 0) && (ldx % 8 == 0);
                NVC_TRY(launch_qmv_affine(dev, q->bits, p, 1));
            }
        }
        return NVC_OK;
    }
    GenericParams g{};
    g.mode = q->mode; g.gs = q->group_size; g.bits = q->bits; g.dtype = dtype; g.transpose = transpose;
    g.scalar_global = global_scale != nullptr; g.expert_global = 0;
    g.x = x; g.w = w; g.scales = scales; g.biases = biases; g.global = global_scale; g.lhs = nullptr; g.rhs = nullptr;
    g.M = M; g.N = N; g.K = K; g.ldx = ldx; g.batch = batch;
    g.x_batch_stride = x_batch_stride; g.w_batch_stride = w_batch_stride; g.s_batch_stride = s_batch_stride;
    g.y = y;
    return launch_generic(dev, g);
}

extern "C" int32_t nvc_gather_qmm(nvc_device *dev, const nvc_quant *q, int32_t dtype, int32_t transpose, const void *x,
                                  const uint32_t *w, const void *scales, const void *biases,
                                  const float *global_scale, const uint32_t *lhs, const uint32_t *rhs,
                                  const int32_t *offsets, int32_t sorted, int64_t rows, int64_t x_batches, int64_t M,
                                  int64_t N, int64_t K, int64_t experts, void *y) {
    NVC_TRY(make_current(dev));
    NVC_TRY(check_product("gather_qmm", q, dtype, transpose, biases, global_scale, M, N, K));
    if (rows < 0 || x_batches < 0 || experts < 0) return set_error(NVC_ERR_INVALID_ARGUMENT, "gather_qmm: negative size");
    if (rows > 0 && (experts < 1 || x_batches < 1 || experts > 0xFFFFFFFFll || x_batches > 0xFFFFFFFFll))
        return set_error(NVC_ERR_INVALID_ARGUMENT, "gather_qmm: %lld rows gathered from %lld weight batches and %lld activation batches",
                         (long long)rows, (long long)experts, (long long)x_batches);
    if (rows == 0 || M == 0 || N == 0) return NVC_OK;
    if (!x || !w || !scales || !y || !rhs) return set_error(NVC_ERR_INVALID_ARGUMENT, "gather_qmm: null operand");
    if (K == 0) {
        NVC_CUDA(cudaMemsetAsync(y, 0, (size_t)(rows * M * N) * dtype_size(dtype), dev->stream));
        return NVC_OK;
    }
    const int64_t w_stride = (transpose ? N : K) * ((transpose ? K : N) * q->bits / 32);
    const int64_t s_stride = (transpose ? N : K) * ((transpose ? K : N) / q->group_size);
    // Sorted rows of one expert multiplied together (the reference's grouped kernel).  The
    // reference's row-count rule chooses between two algorithms with the same result; here it
    // chooses between the tensor-core kernel and the few-row kernel, and shapes the few-row
    // kernel does not take go to the tensor-core kernel whatever the count.
    const bool few_rows_ok = M <= 8 && qmv_affine_eligible(q->mode, q->group_size, q->bits, dtype, transpose, M, N, K, x, K,
                                                           M * K, w, w_stride);
    if (sorted && !lhs && M == 1 && (grouped(rows, experts, dev->row_exact) || !few_rows_ok) &&
        qmm_eligible(q->mode, q->group_size, q->bits, dtype, transpose, rows, N, K, x, K, w)) {
        const int32_t *offs = offsets;
        if (!offs) {
            void *scratch = nullptr;
            NVC_TRY(ensure_scratch(dev, (size_t)experts * sizeof(int32_t), &scratch));
            NVC_TRY(run_sorted_offsets(dev, rhs, rows, experts, (int32_t *)scratch));
            offs = (const int32_t *)scratch;
        }
        QmmParams p{};
        p.mode = q->mode; p.gs = q->group_size; p.bits = q->bits;
        p.x = x; p.w = w; p.scales = scales; p.biases = biases;
        p.global = global_scale; p.expert_global = global_scale != nullptr;
        p.offsets = offs; p.experts = experts;
        p.rows = rows; p.N = N; p.K = K; p.ldx = K; p.y = y;
        return launch_qmm(dev, p);
    }
    if (few_rows_ok) {
        QmvParams p{};
        p.x = x; p.w = w; p.scales = scales; p.biases = biases; p.lhs = lhs; p.rhs = rhs; p.y = y;
        p.N = N; p.K = K; p.ldx = K;
        p.x_batch_stride = M * K; p.w_batch_stride = w_stride; p.s_batch_stride = s_stride;
        p.M = (int32_t)M; p.gs = q->group_size;
        p.x_vec = ((uintptr_t)x % 16 == 0) && (K % 8 == 0);
        p.global = global_scale; p.expert_global = global_scale != nullptr;
        p.experts = (uint32_t)experts; p.x_batches = (uint32_t)x_batches;
        // Row batches beyond the grid limit go in slices.
        for (int64_t r0 = 0; r0 < rows; r0 += 65535) {
            int64_t n = rows - r0 < 65535 ? rows - r0 : 65535;
            QmvParams s = p;
            s.lhs = lhs ? lhs + r0 : nullptr;
            s.rhs = rhs + r0;
            if (!lhs) s.x = (const char *)x + r0 * M * K * dtype_size(dtype);
            s.y = (char *)y + r0 * M * N * dtype_size(dtype);
            NVC_TRY(launch_qmv_affine(dev, qmv_kind(q->mode, q->bits), s, n));
        }
        return NVC_OK;
    }
    GenericParams g{};
    g.mode = q->mode; g.gs = q->group_size; g.bits = q->bits; g.dtype = dtype; g.transpose = transpose;
    g.scalar_global = 0; g.expert_global = global_scale != nullptr;
    g.experts = (uint32_t)experts; g.x_batches = (uint32_t)x_batches;
    g.w = w; g.scales = scales; g.biases = biases; g.global = global_scale;
    g.M = M; g.N = N; g.K = K; g.ldx = K;
    g.x_batch_stride = M * K; g.w_batch_stride = w_stride; g.s_batch_stride = s_stride;
    for (int64_t r0 = 0; r0 < rows; r0 += 65535) {
        int64_t n = rows - r0 < 65535 ? rows - r0 : 65535;
        g.lhs = lhs ? lhs + r0 : nullptr;
        g.rhs = rhs + r0;
        g.x = lhs ? x : (const void *)((const char *)x + r0 * M * K * dtype_size(dtype));
        g.y = (char *)y + r0 * M * N * dtype_size(dtype);
        g.batch = n;
        NVC_TRY(launch_generic(dev, g));
    }
    return NVC_OK;
}

static int32_t ensure_staging(nvc_device *dev, size_t host_bytes, size_t dev_bytes) {
    if (dev->pinned_bytes < host_bytes) {
        NVC_CUDA(cudaStreamSynchronize(dev->stream));
        if (dev->pinned) cudaFreeHost(dev->pinned);
        dev->pinned = nullptr;
        dev->pinned_bytes = 0;
        NVC_CUDA(cudaHostAlloc(&dev->pinned, host_bytes, cudaHostAllocMapped));
        dev->pinned_bytes = host_bytes;
    }
    if (dev->staging_bytes < dev_bytes) {
        NVC_CUDA(cudaStreamSynchronize(dev->stream));
        if (dev->staging) NVC_TRY(dev->pool.free(dev->staging));
        dev->staging = nullptr;
        dev->staging_bytes = 0;
        NVC_TRY(dev->pool.alloc(dev_bytes, &dev->staging));
        dev->staging_bytes = dev_bytes;
    }
    return NVC_OK;
}

extern "C" int32_t nvc_quantized_matmul_host(nvc_device *dev, const nvc_quant *q, int32_t dtype, int32_t transpose,
                                             const void *host_x, const uint32_t *w, const void *scales,
                                             const void *biases, const float *global_scale, int64_t M, int64_t N,
                                             int64_t K, void *host_y) {
    NVC_TRY(make_current(dev));
    NVC_TRY(check_product("quantized_matmul", q, dtype, transpose, biases, global_scale, M, N, K));
    if (M == 0 || N == 0) return NVC_OK;
    if (!host_x || !host_y) return set_error(NVC_ERR_INVALID_ARGUMENT, "quantized_matmul: null host operand");
    const size_t xb = (size_t)(M * K) * dtype_size(dtype), yb = (size_t)(M * N) * dtype_size(dtype);
    const size_t xoff = 0, yoff = (xb + 255) / 256 * 256;
    NVC_TRY(ensure_staging(dev, yoff + yb, yoff + yb));
    char *hp = (char *)dev->pinned, *dp = (char *)dev->staging;
    // Pageable caller memory goes through the pinned block so both copies are asynchronous
    // DMA transfers on the stream; a caller that passes pinned memory skips nothing but a memcpy.
    memcpy(hp + xoff, host_x, xb);
    NVC_CUDA(cudaMemcpyAsync(dp + xoff, hp + xoff, xb, cudaMemcpyHostToDevice, dev->stream));
    // A small result (a decode product: a few KB) is stored by the kernel straight into the pinned
    // block through its device mapping, which saves a copy command and its latency; a large one
    // goes to device memory and comes back as one DMA transfer.
    void *ydev = dp + yoff;
    const bool direct = yb <= 256 * 1024;
    if (direct) NVC_CUDA(cudaHostGetDevicePointer(&ydev, hp + yoff, 0));
    NVC_TRY(nvc_quantized_matmul(dev, q, dtype, transpose, dp + xoff, w, scales, biases, global_scale, M, N, K, K, 1, 0,
                                 0, 0, ydev));
    if (!direct) NVC_CUDA(cudaMemcpyAsync(hp + yoff, dp + yoff, yb, cudaMemcpyDeviceToHost, dev->stream));
    NVC_CUDA(cudaStreamSynchronize(dev->stream));
    memcpy(host_y, hp + yoff, yb);
    return NVC_OK;
}

// The asynchronous form of the host-operand product: nothing waits.  The activations are copied
// into a pinned block and from there to the device on the stream, the kernel follows, and the
// result stays pending -- stored by the kernel straight into the pinned block through its device
// mapping when it is small, copied back on the stream otherwise -- until nvc_synchronize (or any
// call that synchronizes, such as nvc_memcpy_d2h) delivers it into host_y.  This is how the
// reference's evaluator treats GPU results: pending until flush
// (crates/nuvec-core/src/gpu.rs:1772-1795).  host_x may be reused as soon as the call returns;
// host_y must stay valid until the synchronization.
extern "C" int32_t nvc_quantized_matmul_host_async(nvc_device *dev, const nvc_quant *q, int32_t dtype, int32_t transpose,
                                                   const void *host_x, const uint32_t *w, const void *scales,
                                                   const void *biases, const float *global_scale, int64_t M, int64_t N,
                                                   int64_t K, void *host_y) {
    NVC_TRY(make_current(dev));
    NVC_TRY(check_product("quantized_matmul", q, dtype, transpose, biases, global_scale, M, N, K));
    if (M == 0 || N == 0) return NVC_OK;
    if (!host_x || !host_y) return set_error(NVC_ERR_INVALID_ARGUMENT, "quantized_matmul: null host operand");
    if (dev->capturing) return set_error(NVC_ERR_UNSUPPORTED, "quantized_matmul (host operands): not inside a recorded step");
    const size_t xb = (size_t)(M * K) * dtype_size(dtype), yb = (size_t)(M * N) * dtype_size(dtype);
    const size_t xpad = (xb + 255) / 256 * 256, ypad = (yb + 255) / 256 * 256;
    constexpr size_t RING = (size_t)64 << 20;
    if (xpad + ypad > RING)  // too large to stage beside other pending work: the synchronous form
        return nvc_quantized_matmul_host(dev, q, dtype, transpose, host_x, w, scales, biases, global_scale, M, N, K, host_y);
    if (!dev->ring_host) {
        NVC_CUDA(cudaHostAlloc((void **)&dev->ring_host, RING, cudaHostAllocMapped));
        NVC_CUDA(cudaHostGetDevicePointer((void **)&dev->ring_host_dev, dev->ring_host, 0));
        void *d = nullptr;
        NVC_TRY(dev->pool.alloc(RING, &d));
        dev->ring_dev = static_cast<char *>(d);
        dev->ring_bytes = RING;
    }
    if (dev->ring_at + xpad + ypad > dev->ring_bytes) NVC_TRY(nvc_synchronize(dev));  // delivers what is pending, rewinds the blocks
    size_t at;
    {
        std::lock_guard<std::mutex> g(dev->host_mu);
        at = dev->ring_at;
        dev->ring_at += xpad + ypad;
    }
    char *hx = dev->ring_host + at, *hy = hx + xpad, *dx = dev->ring_dev + at, *dy = dx + xpad;
    memcpy(hx, host_x, xb);
    // The activations go to device memory first: every block of the product reads all of them, which
    // over PCIe (reading the pinned block in place) was measured 15 times slower than one copy.
    const void *xdev = dx;
    NVC_CUDA(cudaMemcpyAsync(dx, hx, xb, cudaMemcpyHostToDevice, dev->stream));
    void *ydev = dy;
    const bool direct = yb <= 256 * 1024;
    if (direct) ydev = dev->ring_host_dev + at + xpad;
    NVC_TRY(nvc_quantized_matmul(dev, q, dtype, transpose, xdev, w, scales, biases, global_scale, M, N, K, K, 1, 0, 0, 0, ydev));
    if (!direct) NVC_CUDA(cudaMemcpyAsync(hy, dy, yb, cudaMemcpyDeviceToHost, dev->stream));
    std::lock_guard<std::mutex> g(dev->host_mu);
    dev->pending.push_back({hy, host_y, yb});
    return NVC_OK;
}

// A list of asynchronous host-operand products in one call: what an evaluator that walks a step's
// nodes issues between two flushes.  All activations of the list are packed into the pinned block
// and reach the device in ONE copy (a copy command per product costs more than a decode product
// itself), then the kernels follow back to back; every result is stored by its kernel into the
// pinned block (or copied back when large) and stays pending until the synchronization.  A list
// that does not fit the staging blocks is issued product by product.
// (internal) the list could not be recorded: it has been marked and the call runs once more, unrecorded
static constexpr int32_t HOST_BATCH_AGAIN = 1;

static int32_t host_batch(nvc_device *dev, const nvc_host_product *items, size_t count) {
    if (count && !items) return set_error(NVC_ERR_INVALID_ARGUMENT, "quantized_matmul (host batch): null list");
    if (count == 0) return NVC_OK;
    NVC_TRY(make_current(dev));
    if (dev->capturing) return set_error(NVC_ERR_UNSUPPORTED, "quantized_matmul (host operands): not inside a recorded step");
    constexpr size_t RING = (size_t)64 << 20;
    auto pad = [](size_t n) { return (n + 255) / 256 * 256; };
    size_t xtotal = 0, ytotal = 0;
    for (size_t i = 0; i < count; i++) {
        const nvc_host_product &it = items[i];
        NVC_TRY(check_product("quantized_matmul", &it.quant, it.dtype, it.transpose, it.biases, it.global_scale, it.M, it.N, it.K));
        if ((it.M != 0 && it.N != 0) && (!it.host_x || !it.host_y))
            return set_error(NVC_ERR_INVALID_ARGUMENT, "quantized_matmul (host batch): null host operand in product %zu", i);
        xtotal += pad((size_t)(it.M * it.K) * dtype_size(it.dtype));
        ytotal += pad((size_t)(it.M * it.N) * dtype_size(it.dtype));
    }
    if (xtotal + ytotal > RING) {
        for (size_t i = 0; i < count; i++) {
            const nvc_host_product &it = items[i];
            NVC_TRY(nvc_quantized_matmul_host_async(dev, &it.quant, it.dtype, it.transpose, it.host_x, it.w, it.scales, it.biases,
                                                    it.global_scale, it.M, it.N, it.K, it.host_y));
        }
        return NVC_OK;
    }
    if (!dev->ring_host) {
        NVC_CUDA(cudaHostAlloc((void **)&dev->ring_host, RING, cudaHostAllocMapped));
        NVC_CUDA(cudaHostGetDevicePointer((void **)&dev->ring_host_dev, dev->ring_host, 0));
        void *d = nullptr;
        NVC_TRY(dev->pool.alloc(RING, &d));
        dev->ring_dev = static_cast<char *>(d);
        dev->ring_bytes = RING;
    }
    if (dev->ring_at + xtotal + ytotal > dev->ring_bytes) NVC_TRY(nvc_synchronize(dev));
    size_t at;
    {
        std::lock_guard<std::mutex> g(dev->host_mu);
        at = dev->ring_at;
        dev->ring_at += xtotal + ytotal;
    }
    // activations: packed front to back, one copy
    size_t xo = at;
    for (size_t i = 0; i < count; i++) {
        const size_t xb = (size_t)(items[i].M * items[i].K) * dtype_size(items[i].dtype);
        if (xb) memcpy(dev->ring_host + xo, items[i].host_x, xb);
        xo += pad(xb);
    }
    // A decode loop sends the same list step after step (same weights, same host buffers).  The
    // second time a list arrives its copy and kernels are recorded (the first, unrecorded run has
    // sized every scratch buffer, so nothing allocates while recording); after that one replay
    // stands for the whole list.
    const unsigned char *key = reinterpret_cast<const unsigned char *>(items);
    const size_t key_bytes = count * sizeof(nvc_host_product);
    const bool same_list = dev->batch_key.size() == key_bytes && memcmp(dev->batch_key.data(), key, key_bytes) == 0;
    const bool same = same_list && dev->batch_at == at;
    if (!same_list) dev->batch_norecord = false;
    if (same && dev->batch_exec) {
        NVC_CUDA(cudaGraphLaunch(dev->batch_exec, dev->stream));
        dev->launches += dev->batch_kernels;
        std::lock_guard<std::mutex> g(dev->host_mu);
        dev->pending.insert(dev->pending.end(), dev->batch_results.begin(), dev->batch_results.end());
        return NVC_OK;
    }
    if (dev->batch_exec) {  // a different list: the old recording is of no use any more
        cudaGraphExecDestroy(dev->batch_exec);
        dev->batch_exec = nullptr;
    }
    const bool record = same && !dev->batch_norecord && dev->stream == dev->own_stream;
    if (!same) {
        dev->batch_key.assign(key, key + key_bytes);
        dev->batch_at = at;
    }
    const size_t pending_before = dev->pending.size();
    if (record) {
        NVC_CUDA(cudaStreamBeginCapture(dev->stream, cudaStreamCaptureModeThreadLocal));
        dev->capturing = true;
        dev->captured = 0;
    }
    // (leaves the recording, if one is open, before an error is returned)
    auto finish = [&](int32_t rc) -> int32_t {
        if (!record) return rc;
        dev->capturing = false;
        cudaGraph_t graph = nullptr;
        cudaError_t err = cudaStreamEndCapture(dev->stream, &graph);
        if (rc == NVC_OK && err == cudaSuccess) {
            err = cudaGraphInstantiate(&dev->batch_exec, graph, 0);
            if (err != cudaSuccess) dev->batch_exec = nullptr;
        }
        if (graph) cudaGraphDestroy(graph);
        if (rc != NVC_OK || err != cudaSuccess) {
            // Something in this list does not record (a product that has to grow a scratch buffer,
            // say).  Nothing has run: forget what was queued and let the caller run the list the
            // plain way, now and from now on.
            cudaGetLastError();
            dev->batch_norecord = true;
            std::lock_guard<std::mutex> g(dev->host_mu);
            dev->pending.resize(pending_before);
            return HOST_BATCH_AGAIN;
        }
        dev->batch_kernels = dev->captured;
        {
            std::lock_guard<std::mutex> g(dev->host_mu);
            dev->batch_results.assign(dev->pending.begin() + pending_before, dev->pending.end());
        }
        NVC_CUDA(cudaGraphLaunch(dev->batch_exec, dev->stream));
        return NVC_OK;
    };
    if (xtotal) {
        cudaError_t err = cudaMemcpyAsync(dev->ring_dev + at, dev->ring_host + at, xtotal, cudaMemcpyHostToDevice, dev->stream);
        if (err != cudaSuccess) return finish(cuda_error("cudaMemcpyAsync", err));
    }
    xo = at;
    size_t yo = at + xtotal;
    for (size_t i = 0; i < count; i++) {
        const nvc_host_product &it = items[i];
        const size_t xb = (size_t)(it.M * it.K) * dtype_size(it.dtype), yb = (size_t)(it.M * it.N) * dtype_size(it.dtype);
        if (it.M != 0 && it.N != 0) {
            const bool direct = yb <= 256 * 1024;
            void *ydev = direct ? (void *)(dev->ring_host_dev + yo) : (void *)(dev->ring_dev + yo);
            int32_t rc = nvc_quantized_matmul(dev, &it.quant, it.dtype, it.transpose, dev->ring_dev + xo, it.w, it.scales, it.biases,
                                              it.global_scale, it.M, it.N, it.K, it.K, 1, 0, 0, 0, ydev);
            if (rc != NVC_OK) return finish(rc);
            if (!direct) {
                cudaError_t err = cudaMemcpyAsync(dev->ring_host + yo, dev->ring_dev + yo, yb, cudaMemcpyDeviceToHost, dev->stream);
                if (err != cudaSuccess) return finish(cuda_error("cudaMemcpyAsync", err));
            }
            std::lock_guard<std::mutex> g(dev->host_mu);
            dev->pending.push_back({dev->ring_host + yo, it.host_y, yb});
        }
        xo += pad(xb);
        yo += pad(yb);
    }
    return finish(NVC_OK);
}

extern "C" int32_t nvc_quantized_matmul_host_batch(nvc_device *dev, const nvc_host_product *items, size_t count) {
    int32_t rc = host_batch(dev, items, count);
    if (rc == HOST_BATCH_AGAIN) rc = host_batch(dev, items, count);
    return rc;
}
