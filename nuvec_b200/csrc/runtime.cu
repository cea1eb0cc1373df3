// Device handle, caching allocator, copies, events and error reporting of the CUDA backend.
// Serves the seams the reference's experimental CUDA runtime exposes to its evaluator
// (crates/nuvec-gpu/src/cuda/device.rs:40-227, memory.rs:35-306, error.rs:6-42).
#include "common.cuh"

#include <cstring>

namespace nvc {

static thread_local char g_error[512] = "";

int32_t set_error(int32_t status, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof g_error, fmt, ap);
    va_end(ap);
    return status;
}

int32_t cuda_error(const char *call, cudaError_t err) {
    int32_t status = err == cudaErrorMemoryAllocation ? NVC_ERR_OUT_OF_MEMORY
                     : (err == cudaErrorNoDevice || err == cudaErrorInsufficientDriver) ? NVC_ERR_NO_DEVICE
                                                                                        : NVC_ERR_DRIVER;
    return set_error(status, "%s: %s (%s)", call, cudaGetErrorString(err), cudaGetErrorName(err));
}

int32_t make_current(nvc_device *dev) {
    if (!dev) return set_error(NVC_ERR_INVALID_ARGUMENT, "null device handle");
    int cur = -1;
    if (cudaGetDevice(&cur) == cudaSuccess && cur == dev->ordinal) return NVC_OK;
    NVC_CUDA(cudaSetDevice(dev->ordinal));
    return NVC_OK;
}

int32_t check_launch(nvc_device *dev, const char *kernel) {
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess)
        return set_error(NVC_ERR_DRIVER, "launch of %s failed: %s", kernel, cudaGetErrorString(err));
    if (dev->capturing) dev->captured++;  // counted again at every replay
    else dev->launches++;
    return NVC_OK;
}

int32_t deliver_pending(nvc_device *dev) {
    std::lock_guard<std::mutex> g(dev->host_mu);
    for (const auto &r : dev->pending) std::memcpy(r.host, r.pinned, r.bytes);
    dev->pending.clear();
    dev->ring_at = 0;
    return NVC_OK;
}

int32_t ensure_error_word(nvc_device *dev) {
    if (!dev->error_word) {
        NVC_CUDA(cudaHostAlloc((void **)&dev->error_word, sizeof(int32_t), cudaHostAllocMapped));
        *dev->error_word = 0;
        NVC_CUDA(cudaHostGetDevicePointer((void **)&dev->error_word_dev, dev->error_word, 0));
    }
    return NVC_OK;
}

int32_t check_quant(const char *op, const nvc_quant *q) {
    if (!q) return set_error(NVC_ERR_INVALID_ARGUMENT, "%s: null quantization", op);
    int gs = q->group_size, bits = q->bits;
    if (q->mode == NVC_AFFINE) {
        if (gs != 32 && gs != 64 && gs != 128)
            return set_error(NVC_ERR_INVALID_ARGUMENT, "%s: group size %d is not supported (32, 64 or 128)", op, gs);
        if (!((bits >= 1 && bits <= 6) || bits == 8))
            return set_error(NVC_ERR_INVALID_ARGUMENT, "%s: %d bits are not supported (1, 2, 3, 4, 5, 6 or 8)", op, bits);
        return NVC_OK;
    }
    const char *name = q->mode == NVC_MXFP4 ? "mxfp4" : q->mode == NVC_MXFP8 ? "mxfp8" : q->mode == NVC_NVFP4 ? "nvfp4" : nullptr;
    if (!name) return set_error(NVC_ERR_INVALID_ARGUMENT, "%s: invalid quantization mode %d (affine, mxfp4, mxfp8 or nvfp4)", op, q->mode);
    int eg = q->mode == NVC_NVFP4 ? 16 : 32, eb = q->mode == NVC_MXFP8 ? 8 : 4;
    if (gs != eg) return set_error(NVC_ERR_INVALID_ARGUMENT, "%s: %s quantization requires group size %d but got %d", op, name, eg, gs);
    if (bits != eb) return set_error(NVC_ERR_INVALID_ARGUMENT, "%s: %s quantization requires bits to be %d but got %d", op, name, eb, bits);
    return NVC_OK;
}

// ── pool ───────────────────────────────────────────────────────────────────────────────

// memory.rs:54-60: <= 8 bytes -> 8; below 16 KiB -> next power of two; else whole 16 KiB pages.
size_t Pool::size_class(size_t bytes) {
    if (bytes <= 8) return 8;
    if (bytes < (16u << 10)) {
        size_t c = 8;
        while (c < bytes) c <<= 1;
        return c;
    }
    const size_t page = 16u << 10;
    return (bytes + page - 1) / page * page;
}

int32_t Pool::alloc(size_t bytes, void **out) {
    *out = nullptr;
    if (bytes == 0) bytes = 1;
    size_t cls = size_class(bytes);
    // cudaMalloc returns 256-byte aligned blocks; classes below that are rounded up so every
    // block keeps that alignment when carved by nobody but the driver.
    std::lock_guard<std::mutex> g(mu_);
    auto it = free_.find(cls);
    if (it != free_.end()) {
        *out = it->second;
        free_.erase(it);
        cached_ -= cls;
    } else {
        if (active_ + cls > limit_)
            return set_error(NVC_ERR_OUT_OF_MEMORY, "allocation of %zu bytes exceeds the memory limit (%llu active, limit %llu)",
                             bytes, (unsigned long long)active_, (unsigned long long)limit_);
        cudaError_t err = cudaMalloc(out, cls);
        if (err == cudaErrorMemoryAllocation) {
            // Give cached blocks back to the driver and try once more (memory.rs retries the
            // same way after clearing its cache).
            cudaGetLastError();
            trim_locked(0);
            err = cudaMalloc(out, cls);
        }
        if (err != cudaSuccess) {
            cudaGetLastError();
            *out = nullptr;
            return set_error(NVC_ERR_OUT_OF_MEMORY, "cudaMalloc(%zu): %s", cls, cudaGetErrorString(err));
        }
        allocations_++;
    }
    live_[*out] = cls;
    active_ += cls;
    if (active_ > peak_) peak_ = active_;
    return NVC_OK;
}

int32_t Pool::free(void *ptr) {
    if (!ptr) return NVC_OK;
    std::lock_guard<std::mutex> g(mu_);
    auto it = live_.find(ptr);
    if (it == live_.end()) return set_error(NVC_ERR_INVALID_ARGUMENT, "nvc_free: pointer %p was not allocated by this device handle", ptr);
    size_t cls = it->second;
    live_.erase(it);
    active_ -= cls;
    free_.emplace(cls, ptr);
    cached_ += cls;
    if (cached_ > cache_limit_) trim_locked(cache_limit_);
    return NVC_OK;
}

void Pool::trim_locked(uint64_t target) {
    // Largest blocks first.
    while (cached_ > target && !free_.empty()) {
        auto it = std::prev(free_.end());
        cudaFree(it->second);
        cached_ -= it->first;
        free_.erase(it);
    }
}

int32_t Pool::clear() {
    std::lock_guard<std::mutex> g(mu_);
    trim_locked(0);
    return NVC_OK;
}

void Pool::set_cache_limit(uint64_t b) {
    std::lock_guard<std::mutex> g(mu_);
    cache_limit_ = b;
    if (cached_ > cache_limit_) trim_locked(cache_limit_);
}

void Pool::stats(nvc_mem_stats *out) {
    std::lock_guard<std::mutex> g(mu_);
    out->active = active_;
    out->cached = cached_;
    out->peak = peak_;
    out->limit = limit_;
    out->cache_limit = cache_limit_;
    out->allocations = allocations_;
}

int32_t ensure_scratch(nvc_device *dev, size_t bytes, void **out) {
    if (dev->scratch_bytes < bytes) {
        // Earlier work on the stream may still be using the old block.
        NVC_CUDA(cudaStreamSynchronize(dev->stream));
        if (dev->scratch) NVC_TRY(dev->pool.free(dev->scratch));
        dev->scratch = nullptr;
        dev->scratch_bytes = 0;
        size_t want = bytes < (4u << 20) ? (4u << 20) : bytes;
        NVC_TRY(dev->pool.alloc(want, &dev->scratch));
        dev->scratch_bytes = want;
    }
    *out = dev->scratch;
    return NVC_OK;
}

int32_t ensure_counters(nvc_device *dev, size_t count, uint32_t **out) {
    if (dev->counters_len < count) {
        NVC_CUDA(cudaStreamSynchronize(dev->stream));
        if (dev->counters) NVC_TRY(dev->pool.free(dev->counters));
        dev->counters = nullptr;
        dev->counters_len = 0;
        size_t want = count < 4096 ? 4096 : count;
        void *p = nullptr;
        NVC_TRY(dev->pool.alloc(want * sizeof(uint32_t), &p));
        NVC_CUDA(cudaMemsetAsync(p, 0, want * sizeof(uint32_t), dev->stream));
        dev->counters = (uint32_t *)p;
        dev->counters_len = want;
    }
    *out = dev->counters;
    return NVC_OK;
}

}  // namespace nvc

using namespace nvc;

extern "C" {

void nvc_last_error(char *buf, size_t len) {
    if (!buf || len == 0) return;
    strncpy(buf, g_error, len - 1);
    buf[len - 1] = 0;
}

const char *nvc_version(void) { return "nuvec-b200 0.1 (sm_100a)"; }

int32_t nvc_device_open(int32_t ordinal, nvc_device **out) {
    if (!out) return set_error(NVC_ERR_INVALID_ARGUMENT, "nvc_device_open: null output");
    *out = nullptr;
    int count = 0;
    cudaError_t err = cudaGetDeviceCount(&count);
    if (err != cudaSuccess || count == 0) {
        cudaGetLastError();
        return set_error(NVC_ERR_NO_DEVICE, "no CUDA device (%s)", err == cudaSuccess ? "count is 0" : cudaGetErrorString(err));
    }
    if (ordinal < 0 || ordinal >= count)
        return set_error(NVC_ERR_INVALID_ARGUMENT, "device ordinal %d out of range (%d devices)", ordinal, count);
    nvc_device *dev = new nvc_device();
    dev->ordinal = ordinal;
    err = cudaSetDevice(ordinal);
    if (err == cudaSuccess) err = cudaGetDeviceProperties(&dev->prop, ordinal);
    if (err != cudaSuccess) {
        delete dev;
        return cuda_error("cudaGetDeviceProperties", err);
    }
    if (dev->prop.major != 10) {
        int major = dev->prop.major, minor = dev->prop.minor;
        delete dev;
        return set_error(NVC_ERR_UNSUPPORTED, "device %d is compute capability %d.%d; this library holds sm_100a kernels only", ordinal, major, minor);
    }
    err = cudaStreamCreateWithFlags(&dev->own_stream, cudaStreamNonBlocking);
    if (err != cudaSuccess) {
        delete dev;
        return cuda_error("cudaStreamCreateWithFlags", err);
    }
    dev->stream = dev->own_stream;
    size_t free_b = 0, total_b = 0;
    if (cudaMemGetInfo(&free_b, &total_b) == cudaSuccess) dev->pool.set_limit((uint64_t)(total_b * 0.95));
    *out = dev;
    return NVC_OK;
}

int32_t nvc_device_close(nvc_device *dev) {
    if (!dev) return NVC_OK;
    NVC_TRY(make_current(dev));
    cudaStreamSynchronize(dev->stream);
    if (dev->scratch) dev->pool.free(dev->scratch);
    if (dev->qmm_partials) dev->pool.free(dev->qmm_partials);
    if (dev->qmm_counters) dev->pool.free(dev->qmm_counters);
    if (dev->counters) dev->pool.free(dev->counters);
    if (dev->ring_dev) dev->pool.free(dev->ring_dev);
    if (dev->batch_exec) cudaGraphExecDestroy(dev->batch_exec);
    if (dev->ring_host) cudaFreeHost(dev->ring_host);
    if (dev->staging) dev->pool.free(dev->staging);
    if (dev->pinned) cudaFreeHost(dev->pinned);
    if (dev->error_word) cudaFreeHost(dev->error_word);
    dev->pool.clear();
    cudaStreamDestroy(dev->own_stream);
    delete dev;
    return NVC_OK;
}

int32_t nvc_device_info(nvc_device *dev, nvc_info *out) {
    if (!dev || !out) return set_error(NVC_ERR_INVALID_ARGUMENT, "nvc_device_info: null argument");
    memset(out, 0, sizeof *out);
    memcpy(out->name, dev->prop.name, sizeof out->name - 1);  // zeroed above: always terminated
    out->cc_major = dev->prop.major;
    out->cc_minor = dev->prop.minor;
    out->multiprocessors = dev->prop.multiProcessorCount;
    out->total_memory = dev->prop.totalGlobalMem;
    out->l2_bytes = (uint64_t)dev->prop.l2CacheSize;
    int drv = 0;
    cudaDriverGetVersion(&drv);
    out->driver_version = drv;
    return NVC_OK;
}

int32_t nvc_synchronize(nvc_device *dev) {
    NVC_TRY(make_current(dev));
    NVC_CUDA(cudaStreamSynchronize(dev->stream));
    deliver_pending(dev);
    if (dev->error_word && *dev->error_word != 0) {
        *dev->error_word = 0;
        // A kernel that gave up may have left arrival counters half-counted: rearm them, so that
        // the next product starts clean.
        if (dev->counters) cudaMemsetAsync(dev->counters, 0, dev->counters_len * sizeof(uint32_t), dev->stream);
        if (dev->qmm_counters) cudaMemsetAsync(dev->qmm_counters, 0, dev->qmm_counters_len * sizeof(uint32_t), dev->stream);
        cudaStreamSynchronize(dev->stream);
        return set_error(NVC_ERR_DRIVER, "a kernel gave up waiting (on its pipeline, or on the other ranks of a fused gather); results of the last work are invalid");
    }
    return NVC_OK;
}

int32_t nvc_device_set_stream(nvc_device *dev, void *cuda_stream) {
    NVC_TRY(make_current(dev));
    NVC_CUDA(cudaStreamSynchronize(dev->stream));
    dev->stream = cuda_stream ? (cudaStream_t)cuda_stream : dev->own_stream;
    return NVC_OK;
}

void *nvc_device_stream(nvc_device *dev) { return dev ? (void *)dev->stream : nullptr; }
uint64_t nvc_launch_count(nvc_device *dev) { return dev ? dev->launches : 0; }

int32_t nvc_alloc(nvc_device *dev, size_t bytes, void **out) {
    if (!out) return set_error(NVC_ERR_INVALID_ARGUMENT, "nvc_alloc: null output");
    NVC_TRY(make_current(dev));
    return dev->pool.alloc(bytes, out);
}

int32_t nvc_free(nvc_device *dev, void *ptr) {
    NVC_TRY(make_current(dev));
    return dev->pool.free(ptr);
}

int32_t nvc_memcpy_h2d(nvc_device *dev, void *dst, const void *src, size_t bytes) {
    NVC_TRY(make_current(dev));
    if (bytes == 0) return NVC_OK;
    NVC_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, dev->stream));
    return NVC_OK;
}

int32_t nvc_memcpy_d2h(nvc_device *dev, void *dst, const void *src, size_t bytes) {
    NVC_TRY(make_current(dev));
    if (bytes == 0) return NVC_OK;
    NVC_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, dev->stream));
    // A host read must see the data: the reference's CPU access waits for GPU work
    // (crates/nuvec-core/src/buffer.rs:204-212).
    return nvc_synchronize(dev);
}

int32_t nvc_memcpy_d2d(nvc_device *dev, void *dst, const void *src, size_t bytes) {
    NVC_TRY(make_current(dev));
    if (bytes == 0) return NVC_OK;
    NVC_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, dev->stream));
    return NVC_OK;
}

int32_t nvc_memset(nvc_device *dev, void *dst, int value, size_t bytes) {
    NVC_TRY(make_current(dev));
    if (bytes == 0) return NVC_OK;
    NVC_CUDA(cudaMemsetAsync(dst, value, bytes, dev->stream));
    return NVC_OK;
}

int32_t nvc_host_alloc(size_t bytes, void **out) {
    if (!out) return set_error(NVC_ERR_INVALID_ARGUMENT, "nvc_host_alloc: null output");
    NVC_CUDA(cudaHostAlloc(out, bytes ? bytes : 1, cudaHostAllocDefault));
    return NVC_OK;
}

int32_t nvc_host_free(void *ptr) {
    if (ptr) NVC_CUDA(cudaFreeHost(ptr));
    return NVC_OK;
}

int32_t nvc_mem_stats_get(nvc_device *dev, nvc_mem_stats *out) {
    if (!dev || !out) return set_error(NVC_ERR_INVALID_ARGUMENT, "nvc_mem_stats_get: null argument");
    dev->pool.stats(out);
    return NVC_OK;
}

int32_t nvc_set_memory_limit(nvc_device *dev, uint64_t bytes) {
    if (!dev) return set_error(NVC_ERR_INVALID_ARGUMENT, "null device handle");
    dev->pool.set_limit(bytes);
    return NVC_OK;
}

int32_t nvc_set_cache_limit(nvc_device *dev, uint64_t bytes) {
    NVC_TRY(make_current(dev));
    NVC_CUDA(cudaStreamSynchronize(dev->stream));
    dev->pool.set_cache_limit(bytes);
    return NVC_OK;
}

int32_t nvc_clear_cache(nvc_device *dev) {
    NVC_TRY(make_current(dev));
    NVC_CUDA(cudaStreamSynchronize(dev->stream));
    return dev->pool.clear();
}

int32_t nvc_reset_peak(nvc_device *dev) {
    if (!dev) return set_error(NVC_ERR_INVALID_ARGUMENT, "null device handle");
    dev->pool.reset_peak();
    return NVC_OK;
}

int32_t nvc_event_create(nvc_device *dev, nvc_event **out) {
    if (!out) return set_error(NVC_ERR_INVALID_ARGUMENT, "nvc_event_create: null output");
    NVC_TRY(make_current(dev));
    nvc_event *e = new nvc_event();
    e->ordinal = dev->ordinal;
    cudaError_t err = cudaEventCreate(&e->ev);
    if (err != cudaSuccess) {
        delete e;
        return cuda_error("cudaEventCreate", err);
    }
    *out = e;
    return NVC_OK;
}

int32_t nvc_event_destroy(nvc_event *ev) {
    if (!ev) return NVC_OK;
    cudaEventDestroy(ev->ev);
    delete ev;
    return NVC_OK;
}

int32_t nvc_event_record(nvc_device *dev, nvc_event *ev) {
    if (!ev) return set_error(NVC_ERR_INVALID_ARGUMENT, "nvc_event_record: null event");
    NVC_TRY(make_current(dev));
    NVC_CUDA(cudaEventRecord(ev->ev, dev->stream));
    return NVC_OK;
}

int32_t nvc_event_synchronize(nvc_event *ev) {
    if (!ev) return set_error(NVC_ERR_INVALID_ARGUMENT, "nvc_event_synchronize: null event");
    NVC_CUDA(cudaEventSynchronize(ev->ev));
    return NVC_OK;
}

int32_t nvc_event_elapsed_ms(nvc_event *start, nvc_event *stop, float *out_ms) {
    if (!start || !stop || !out_ms) return set_error(NVC_ERR_INVALID_ARGUMENT, "nvc_event_elapsed_ms: null argument");
    NVC_CUDA(cudaEventElapsedTime(out_ms, start->ev, stop->ev));
    return NVC_OK;
}

int32_t nvc_graph_begin(nvc_device *dev) {
    NVC_TRY(make_current(dev));
    if (dev->capturing) return set_error(NVC_ERR_INVALID_ARGUMENT, "nvc_graph_begin: already recording");
    NVC_CUDA(cudaStreamBeginCapture(dev->stream, cudaStreamCaptureModeThreadLocal));
    dev->capturing = true;
    dev->captured = 0;
    return NVC_OK;
}

int32_t nvc_graph_end(nvc_device *dev, nvc_graph **out) {
    if (!out) return set_error(NVC_ERR_INVALID_ARGUMENT, "nvc_graph_end: null output");
    *out = nullptr;
    NVC_TRY(make_current(dev));
    if (!dev->capturing) return set_error(NVC_ERR_INVALID_ARGUMENT, "nvc_graph_end: not recording");
    dev->capturing = false;
    cudaGraph_t graph = nullptr;
    NVC_CUDA(cudaStreamEndCapture(dev->stream, &graph));
    nvc_graph *g = new nvc_graph();
    cudaError_t err = cudaGraphInstantiate(&g->exec, graph, 0);
    size_t nodes = 0;
    cudaGraphGetNodes(graph, nullptr, &nodes);
    g->nodes = nodes;
    g->kernels = dev->captured;
    cudaGraphDestroy(graph);
    if (err != cudaSuccess) {
        delete g;
        return cuda_error("cudaGraphInstantiate", err);
    }
    *out = g;
    return NVC_OK;
}

int32_t nvc_graph_launch(nvc_device *dev, nvc_graph *graph) {
    if (!graph) return set_error(NVC_ERR_INVALID_ARGUMENT, "nvc_graph_launch: null graph");
    NVC_TRY(make_current(dev));
    NVC_CUDA(cudaGraphLaunch(graph->exec, dev->stream));
    dev->launches += graph->kernels;
    return NVC_OK;
}

int32_t nvc_graph_destroy(nvc_graph *graph) {
    if (!graph) return NVC_OK;
    cudaGraphExecDestroy(graph->exec);
    delete graph;
    return NVC_OK;
}

}  // extern "C"
