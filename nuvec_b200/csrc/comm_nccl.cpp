// NCCL communicator behind the reference's `Communicator` trait
// (crates/nuvec-core/src/distributed.rs:43-83): rank/size, all_gather, all_reduce (sum, max, min),
// send, recv, health; initialisation under a host-side time limit.
// The reference's transports are a TCP ring and RDMA between Macs
// (crates/nuvec-distributed/src/ring.rs:868-889); on B200 the same byte-level contract is
// served by NCCL over NVLink/NVSwitch, stream-ordered after the kernels.
//
// NCCL is loaded at first use with dlopen, so the library has no link-time dependency on it and
// a process that already holds an NCCL (for example through its tensor framework) shares that
// copy instead of loading a second one.
#include <dlfcn.h>
#include <nccl.h>

#include <chrono>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <thread>

#include "common.cuh"

namespace {

struct Api {
    void *handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommInitRankConfig)(ncclComm_t *, int, ncclUniqueId, int, ncclConfig_t *) = nullptr;
    ncclResult_t (*Send)(const void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Recv)(void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t *) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
    const char *(*GetLastError)(ncclComm_t) = nullptr;
};

Api g_api;
std::once_flag g_once;
char g_load_error[256] = "";

void load_api() {
    const char *names[] = {getenv("NUVEC_NCCL_LIBRARY"), "libnccl.so.2", "libnccl.so"};
    for (const char *n : names) {
        if (!n || !*n) continue;
        g_api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (g_api.handle) break;
    }
    if (!g_api.handle) {
        snprintf(g_load_error, sizeof g_load_error, "cannot load libnccl.so.2: %s", dlerror());
        return;
    }
#define NVC_SYM(field, name)                                                       \
    g_api.field = reinterpret_cast<decltype(g_api.field)>(dlsym(g_api.handle, name)); \
    if (!g_api.field) snprintf(g_load_error, sizeof g_load_error, "libnccl lacks %s", name);
    NVC_SYM(GetUniqueId, "ncclGetUniqueId")
    NVC_SYM(CommInitRank, "ncclCommInitRank")
    NVC_SYM(CommInitRankConfig, "ncclCommInitRankConfig")
    NVC_SYM(Send, "ncclSend")
    NVC_SYM(Recv, "ncclRecv")
    NVC_SYM(AllGather, "ncclAllGather")
    NVC_SYM(AllReduce, "ncclAllReduce")
    NVC_SYM(CommGetAsyncError, "ncclCommGetAsyncError")
    NVC_SYM(CommAbort, "ncclCommAbort")
    NVC_SYM(CommDestroy, "ncclCommDestroy")
    NVC_SYM(GetErrorString, "ncclGetErrorString")
#undef NVC_SYM
    g_api.GetLastError = reinterpret_cast<decltype(g_api.GetLastError)>(dlsym(g_api.handle, "ncclGetLastError"));
}

int32_t api_ready() {
    std::call_once(g_once, load_api);
    if (g_load_error[0]) return nvc::set_error(NVC_ERR_COMM, "%s", g_load_error);
    return NVC_OK;
}

int32_t nccl_error(const char *call, ncclResult_t r) {
    return nvc::set_error(NVC_ERR_COMM, "%s: %s", call, g_api.GetErrorString ? g_api.GetErrorString(r) : "NCCL error");
}

}  // namespace

struct nvc_comm {
    ncclComm_t comm = nullptr;
    nvc_device *dev = nullptr;
    int rank = 0, size = 1;
};

#define NVC_NCCL(call)                                        \
    do {                                                      \
        ncclResult_t r__ = (call);                            \
        if (r__ != ncclSuccess) return nccl_error(#call, r__); \
    } while (0)

// A communicator initialised without blocking stays in that mode: every call may answer "in
// progress", which is waited out here (bounded by the communicator's own watchdog).
static ncclResult_t settle(nvc_comm *comm, ncclResult_t r) {
    while (r == ncclInProgress) {
        ncclResult_t state = ncclSuccess;
        ncclResult_t q = g_api.CommGetAsyncError(comm->comm, &state);
        if (q != ncclSuccess) return q;
        if (state != ncclInProgress) return state;
        std::this_thread::yield();
    }
    return r;
}

extern "C" {

int32_t nvc_comm_unique_id(uint8_t out_id[128]) {
    NVC_TRY(api_ready());
    static_assert(sizeof(ncclUniqueId) == 128, "the ABI carries the id as 128 bytes");
    ncclUniqueId id;
    NVC_NCCL(g_api.GetUniqueId(&id));
    memcpy(out_id, &id, 128);
    return NVC_OK;
}

int32_t nvc_comm_init_timeout(nvc_device *dev, int32_t rank, int32_t size, const uint8_t id[128], int64_t timeout_ms,
                              nvc_comm **out) {
    if (!out || !id) return nvc::set_error(NVC_ERR_INVALID_ARGUMENT, "nvc_comm_init: null argument");
    *out = nullptr;
    if (size < 1 || rank < 0 || rank >= size)
        return nvc::set_error(NVC_ERR_INVALID_ARGUMENT, "nvc_comm_init: rank %d of %d", rank, size);
    NVC_TRY(nvc::make_current(dev));
    NVC_TRY(api_ready());
    if (timeout_ms <= 0) {
        const char *e = getenv("NUVEC_DISTRIBUTED_TIMEOUT");  // seconds, as in the reference
        const double secs = e && *e ? atof(e) : 120.0;
        timeout_ms = secs > 0 ? (int64_t)(secs * 1000.0) : 120000;
    }
    ncclUniqueId uid;
    memcpy(&uid, id, 128);
    nvc_comm *c = new nvc_comm();
    c->dev = dev;
    c->rank = rank;
    c->size = size;
    // Non-blocking initialisation: the call returns at once and the communicator reports
    // "in progress" until every rank has joined, so the wait is this loop's, with a limit.
    ncclConfig_t config = NCCL_CONFIG_INITIALIZER;
    config.blocking = 0;
    ncclResult_t r = g_api.CommInitRankConfig(&c->comm, size, uid, rank, &config);
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
    while (r == ncclInProgress || (r == ncclSuccess && c->comm)) {
        ncclResult_t state = ncclSuccess;
        ncclResult_t q = g_api.CommGetAsyncError(c->comm, &state);
        if (q != ncclSuccess) { r = q; break; }
        if (state != ncclInProgress) { r = state; break; }
        if (std::chrono::steady_clock::now() >= deadline) {
            if (c->comm) g_api.CommAbort(c->comm);
            delete c;
            return nvc::set_error(NVC_ERR_COMM, "nvc_comm_init: rank %d of %d gave up after %lld ms: not every rank joined",
                                  rank, size, (long long)timeout_ms);
        }
        std::this_thread::sleep_for(std::chrono::milliseconds(1));
    }
    if (r != ncclSuccess) {
        if (c->comm) g_api.CommAbort(c->comm);
        delete c;
        return nccl_error("ncclCommInitRankConfig", r);
    }
    *out = c;
    return NVC_OK;
}

int32_t nvc_comm_init(nvc_device *dev, int32_t rank, int32_t size, const uint8_t id[128], nvc_comm **out) {
    return nvc_comm_init_timeout(dev, rank, size, id, 0, out);
}

int32_t nvc_comm_rank(nvc_comm *comm) { return comm ? comm->rank : -1; }
int32_t nvc_comm_size(nvc_comm *comm) { return comm ? comm->size : -1; }

int32_t nvc_all_gather(nvc_comm *comm, const void *send, void *recv, size_t bytes_per_rank) {
    if (!comm) return nvc::set_error(NVC_ERR_INVALID_ARGUMENT, "nvc_all_gather: null communicator");
    NVC_TRY(nvc::make_current(comm->dev));
    if (bytes_per_rank == 0) return NVC_OK;
    NVC_NCCL(settle(comm, g_api.AllGather(send, recv, bytes_per_rank, ncclUint8, comm->comm, comm->dev->stream)));
    return NVC_OK;
}

int32_t nvc_send(nvc_comm *comm, const void *buf, size_t bytes, int32_t peer) {
    if (!comm) return nvc::set_error(NVC_ERR_INVALID_ARGUMENT, "nvc_send: null communicator");
    if (peer < 0 || peer >= comm->size || peer == comm->rank)
        return nvc::set_error(NVC_ERR_INVALID_ARGUMENT, "nvc_send: rank %d sends to rank %d of %d", comm->rank, peer, comm->size);
    NVC_TRY(nvc::make_current(comm->dev));
    if (bytes == 0) return NVC_OK;
    NVC_NCCL(settle(comm, g_api.Send(buf, bytes, ncclUint8, peer, comm->comm, comm->dev->stream)));
    return NVC_OK;
}

int32_t nvc_recv(nvc_comm *comm, void *buf, size_t bytes, int32_t peer) {
    if (!comm) return nvc::set_error(NVC_ERR_INVALID_ARGUMENT, "nvc_recv: null communicator");
    if (peer < 0 || peer >= comm->size || peer == comm->rank)
        return nvc::set_error(NVC_ERR_INVALID_ARGUMENT, "nvc_recv: rank %d receives from rank %d of %d", comm->rank, peer, comm->size);
    NVC_TRY(nvc::make_current(comm->dev));
    if (bytes == 0) return NVC_OK;
    NVC_NCCL(settle(comm, g_api.Recv(buf, bytes, ncclUint8, peer, comm->comm, comm->dev->stream)));
    return NVC_OK;
}

int32_t nvc_all_reduce_sum(nvc_comm *comm, int32_t dtype, void *buf, size_t count) {
    return nvc_all_reduce(comm, NVC_REDUCE_SUM, dtype, buf, count);
}

int32_t nvc_all_reduce(nvc_comm *comm, int32_t op, int32_t dtype, void *buf, size_t count) {
    if (!comm) return nvc::set_error(NVC_ERR_INVALID_ARGUMENT, "nvc_all_reduce: null communicator");
    if (op != NVC_REDUCE_SUM && op != NVC_REDUCE_MAX && op != NVC_REDUCE_MIN)
        return nvc::set_error(NVC_ERR_INVALID_ARGUMENT, "nvc_all_reduce: unknown operation %d", op);
    const ncclRedOp_t rop = op == NVC_REDUCE_SUM ? ncclSum : op == NVC_REDUCE_MAX ? ncclMax : ncclMin;
    NVC_TRY(nvc::make_current(comm->dev));
    ncclDataType_t t;
    switch (dtype) {
    case NVC_F32: t = ncclFloat32; break;
    case NVC_F16: t = ncclFloat16; break;
    case NVC_BF16: t = ncclBfloat16; break;
    case NVC_I32: t = ncclInt32; break;
    default: return nvc::set_error(NVC_ERR_UNSUPPORTED, "all_reduce: unsupported dtype %d", dtype);
    }
    if (count == 0) return NVC_OK;
    NVC_NCCL(settle(comm, g_api.AllReduce(buf, buf, count, t, rop, comm->comm, comm->dev->stream)));
    return NVC_OK;
}

int32_t nvc_comm_health(nvc_comm *comm) {
    if (!comm) return nvc::set_error(NVC_ERR_INVALID_ARGUMENT, "nvc_comm_health: null communicator");
    ncclResult_t async = ncclSuccess;
    NVC_NCCL(g_api.CommGetAsyncError(comm->comm, &async));
    if (async != ncclSuccess && async != ncclInProgress) return nccl_error("asynchronous NCCL error", async);
    return NVC_OK;
}

int32_t nvc_comm_abort(nvc_comm *comm) {
    if (!comm) return NVC_OK;
    if (comm->comm) g_api.CommAbort(comm->comm);
    delete comm;
    return NVC_OK;
}

int32_t nvc_comm_destroy(nvc_comm *comm) {
    if (!comm) return NVC_OK;
    if (comm->comm) g_api.CommDestroy(comm->comm);
    delete comm;
    return NVC_OK;
}

}  // extern "C"
