// Symmetric regions and the peer group of the fused "sharded product + gather": each rank owns a
// region of device memory that the other ranks of the node map through CUDA IPC, and the few-row
// kernel stores its slice of the result into every region (NVLink peer stores) instead of
// handing it to a collective.  Replaces quantized_matmul followed by Communicator::all_gather
// (crates/nuvec-core/src/distributed.rs:52, 695-700) for the decode products.
#include "qmv.cuh"

#include <cstring>

struct nvc_peer_group {
    nvc_device *dev = nullptr;
    nvc::PeerTable host{};
    nvc::PeerTable *table = nullptr;  // device copy
    size_t region_bytes = 0;          // size of every rank's region
};

static size_t round256(size_t n) { return (n + 255) / 256 * 256; }

extern "C" size_t nvc_gather_footprint(int32_t size, int64_t M, int64_t N_local) {
    if (size < 1 || M < 1 || N_local < 1) return 0;
    const size_t per = (size_t)M * (size_t)N_local;
    return round256((size_t)size * per * 2) + round256(2 * (size_t)size * per * 8);
}

extern "C" size_t nvc_all_sum_footprint(int32_t size, int64_t M, int64_t N) {
    if (size < 1 || M < 1 || N < 1) return 0;
    return round256(2 * (size_t)size * (size_t)M * (size_t)N * 8);
}

extern "C" int32_t nvc_symm_alloc(nvc_device *dev, size_t bytes, void **out_ptr, nvc_ipc_handle *out_handle) {
    using namespace nvc;
    NVC_TRY(make_current(dev));
    if (!out_ptr || !out_handle || bytes < NVC_SYMM_RESERVED)
        return set_error(NVC_ERR_INVALID_ARGUMENT, "symm_alloc: needs at least %d bytes and both outputs", NVC_SYMM_RESERVED);
    static_assert(sizeof(cudaIpcMemHandle_t) <= sizeof(nvc_ipc_handle), "handle size");
    void *ptr = nullptr;
    // cudaMalloc directly: an IPC handle names a whole allocation, not a block of the pool
    NVC_CUDA(cudaMalloc(&ptr, bytes));
    NVC_CUDA(cudaMemset(ptr, 0, bytes));
    cudaIpcMemHandle_t h;
    cudaError_t err = cudaIpcGetMemHandle(&h, ptr);
    if (err != cudaSuccess) {
        cudaFree(ptr);
        return cuda_error("cudaIpcGetMemHandle", err);
    }
    std::memset(out_handle, 0, sizeof *out_handle);
    std::memcpy(out_handle->bytes, &h, sizeof h);
    *out_ptr = ptr;
    return NVC_OK;
}

extern "C" int32_t nvc_symm_open(nvc_device *dev, const nvc_ipc_handle *handle, void **out_peer_ptr) {
    using namespace nvc;
    NVC_TRY(make_current(dev));
    if (!handle || !out_peer_ptr) return set_error(NVC_ERR_INVALID_ARGUMENT, "symm_open: null argument");
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle->bytes, sizeof h);
    NVC_CUDA(cudaIpcOpenMemHandle(out_peer_ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return NVC_OK;
}

extern "C" int32_t nvc_symm_close(nvc_device *dev, void *peer_ptr) {
    using namespace nvc;
    NVC_TRY(make_current(dev));
    if (peer_ptr) NVC_CUDA(cudaIpcCloseMemHandle(peer_ptr));
    return NVC_OK;
}

extern "C" int32_t nvc_symm_free(nvc_device *dev, void *ptr) {
    using namespace nvc;
    NVC_TRY(make_current(dev));
    if (ptr) NVC_CUDA(cudaFree(ptr));
    return NVC_OK;
}

extern "C" int32_t nvc_peer_group_create(nvc_device *dev, int32_t rank, int32_t size, void *const *region_bases,
                                         size_t region_bytes, nvc_peer_group **out) {
    using namespace nvc;
    NVC_TRY(make_current(dev));
    if (!region_bases || !out || size < 1 || size > 16 || rank < 0 || rank >= size)
        return set_error(NVC_ERR_INVALID_ARGUMENT, "peer_group_create: rank %d of %d (1 to 16 ranks)", rank, size);
    if (region_bytes < NVC_SYMM_RESERVED)
        return set_error(NVC_ERR_INVALID_ARGUMENT, "peer_group_create: regions of %zu bytes (at least %d)", region_bytes, NVC_SYMM_RESERVED);
    for (int i = 0; i < size; i++)
        if (!region_bases[i]) return set_error(NVC_ERR_INVALID_ARGUMENT, "peer_group_create: region %d is null", i);
    nvc_peer_group *g = new nvc_peer_group;
    g->dev = dev;
    for (int i = 0; i < size; i++) g->host.base[i] = region_bases[i];
    g->host.rank = rank;
    g->host.size = size;
    g->region_bytes = region_bytes;
    void *t = nullptr;
    int32_t rc = dev->pool.alloc(sizeof(PeerTable), &t);
    if (rc != NVC_OK) {
        delete g;
        return rc;
    }
    cudaError_t err = cudaMemcpy(t, &g->host, sizeof(PeerTable), cudaMemcpyHostToDevice);
    if (err != cudaSuccess) {
        dev->pool.free(t);
        delete g;
        return cuda_error("cudaMemcpy", err);
    }
    g->table = static_cast<PeerTable *>(t);
    *out = g;
    return NVC_OK;
}

extern "C" int32_t nvc_peer_group_destroy(nvc_peer_group *group) {
    using namespace nvc;
    if (!group) return NVC_OK;
    NVC_TRY(make_current(group->dev));
    cudaStreamSynchronize(group->dev->stream);
    if (group->table) group->dev->pool.free(group->table);
    delete group;
    return NVC_OK;
}

// Checks shared by the two fused collectives; fills the product's parameters.
static int32_t fused_params(const char *op, nvc_device *dev, nvc_peer_group *group, const nvc_quant *q, const void *x,
                            const uint32_t *w, const void *scales, const void *biases, int64_t M, int64_t N, int64_t K,
                            nvc::QmvParams &p) {
    using namespace nvc;
    NVC_TRY(check_quant(op, q));
    if (!group || group->dev != dev) return set_error(NVC_ERR_INVALID_ARGUMENT, "%s: the group belongs to another device", op);
    if (q->mode != NVC_AFFINE || !biases) return set_error(NVC_ERR_UNSUPPORTED, "%s: affine weights with biases only", op);
    if (M < 1 || N < 1 || K < 1 || K % q->group_size != 0)
        return set_error(NVC_ERR_INVALID_ARGUMENT, "%s: invalid shape [%lld, %lld] x [%lld, %lld]", op, (long long)M, (long long)K,
                         (long long)N, (long long)K);
    if (!x || !w || !scales) return set_error(NVC_ERR_INVALID_ARGUMENT, "%s: null operand", op);
    if (!qmv_affine_eligible(q->mode, q->group_size, q->bits, NVC_BF16, 1, M, N, K, x, K, 0, w, 0))
        return set_error(NVC_ERR_UNSUPPORTED,
                         "%s: takes bfloat16 x with 1 to 8 rows and 2-, 3-, 4-, 6- or 8-bit weights whose rows are a whole "
                         "number of iterations (got M = %lld, K = %lld, %d bits)", op, (long long)M, (long long)K, q->bits);
    NVC_TRY(ensure_error_word(dev));
    p.x = x; p.w = w; p.scales = scales; p.biases = biases; p.lhs = nullptr; p.rhs = nullptr; p.y = nullptr;
    p.N = N; p.K = K; p.ldx = K;
    p.x_batch_stride = 0; p.w_batch_stride = 0; p.s_batch_stride = 0;
    p.M = (int32_t)M; p.gs = q->group_size;
    p.x_vec = ((uintptr_t)x % 16 == 0) && (K % 8 == 0);
    p.peer = group->table;
    p.peer_rank = group->host.rank;
    p.peer_size = group->host.size;
    p.error = dev->error_word_dev;
    return NVC_OK;
}

// True when [a, a + na) and [b, b + nb) share a byte.
static bool overlaps(const void *a, size_t na, const void *b, size_t nb) {
    const uintptr_t a0 = (uintptr_t)a, b0 = (uintptr_t)b;
    return a0 < b0 + nb && b0 < a0 + na;
}

extern "C" int32_t nvc_quantized_matmul_gather(nvc_device *dev, nvc_peer_group *group, const nvc_quant *q, const void *x,
                                               const uint32_t *w, const void *scales, const void *biases, int64_t M,
                                               int64_t N_local, int64_t K, size_t out_offset) {
    using namespace nvc;
    NVC_TRY(make_current(dev));
    QmvParams p{};
    NVC_TRY(fused_params("quantized_matmul_gather", dev, group, q, x, w, scales, biases, M, N_local, K, p));
    const size_t foot = nvc_gather_footprint(group->host.size, M, N_local);
    if (out_offset < NVC_SYMM_RESERVED || out_offset % 256 != 0 || out_offset + foot > group->region_bytes)
        return set_error(NVC_ERR_INVALID_ARGUMENT,
                         "quantized_matmul_gather: offset %zu with a footprint of %zu bytes does not fit a region of %zu bytes "
                         "(offsets start at %d and are multiples of 256)", out_offset, foot, group->region_bytes, NVC_SYMM_RESERVED);
    char *own = static_cast<char *>(group->host.base[group->host.rank]);
    if (overlaps(x, (size_t)(M * K) * 2, own + out_offset, foot))
        return set_error(NVC_ERR_INVALID_ARGUMENT, "quantized_matmul_gather: the activations overlap the product's own buffers");
    p.peer_mode = 1;
    p.peer_out_offset = out_offset;
    p.peer_ll_offset = out_offset + round256((size_t)group->host.size * (size_t)(M * N_local) * 2);
    return launch_qmv_affine(dev, q->bits, p, 1);
}

extern "C" int32_t nvc_quantized_matmul_all_sum(nvc_device *dev, nvc_peer_group *group, const nvc_quant *q, const void *x,
                                                const uint32_t *w, const void *scales, const void *biases, int64_t M,
                                                int64_t N, int64_t K_local, void *y, size_t scratch_offset) {
    using namespace nvc;
    NVC_TRY(make_current(dev));
    QmvParams p{};
    NVC_TRY(fused_params("quantized_matmul_all_sum", dev, group, q, x, w, scales, biases, M, N, K_local, p));
    if (!y) return set_error(NVC_ERR_INVALID_ARGUMENT, "quantized_matmul_all_sum: null output");
    const size_t foot = nvc_all_sum_footprint(group->host.size, M, N);
    if (scratch_offset < NVC_SYMM_RESERVED || scratch_offset % 256 != 0 || scratch_offset + foot > group->region_bytes)
        return set_error(NVC_ERR_INVALID_ARGUMENT,
                         "quantized_matmul_all_sum: offset %zu with a footprint of %zu bytes does not fit a region of %zu bytes "
                         "(offsets start at %d and are multiples of 256)", scratch_offset, foot, group->region_bytes, NVC_SYMM_RESERVED);
    char *own = static_cast<char *>(group->host.base[group->host.rank]);
    if (overlaps(x, (size_t)(M * K_local) * 2, own + scratch_offset, foot) || overlaps(y, (size_t)(M * N) * 2, own + scratch_offset, foot))
        return set_error(NVC_ERR_INVALID_ARGUMENT, "quantized_matmul_all_sum: an operand overlaps the product's packet areas");
    p.y = y;
    p.peer_mode = 2;
    p.peer_out_offset = 0;
    p.peer_ll_offset = scratch_offset;
    return launch_qmv_affine(dev, q->bits, p, 1);
}
