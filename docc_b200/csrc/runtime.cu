// Context, memory pool, transfers and status reporting of the docc_b200 runtime.
//
// Replaces what docc's CUDA target emits around every offloaded region:
// cudaSetDevice(0) (cpp_code_generator.cpp:191,218), cudaMalloc / cudaMemcpy / cudaFree per
// argument (cuda_data_offloading_node.cpp:139-173) and cudaDeviceSynchronize (cuda.cpp:93-103).
#include <map>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "common.cuh"

namespace docc_b200 {

namespace {
thread_local char tls_error[512] = "";
thread_local Ctx tls_ctx[16];

// The pool is stream ordered: a freed block remembers the stream it was freed on and an event recorded there at the
// moment of the free. The next owner gets it at once when it allocates on the same stream (work queued there runs
// after the previous owner's), and otherwise its stream is made to wait for the event (cudaStreamWaitEvent), so a
// kernel of the previous owner that is still running can never overlap the new owner's work. Nothing blocks the host.
struct FreeBlock {
    void* ptr;
    cudaStream_t stream;  // stream the block was freed on
    cudaEvent_t event;    // recorded on that stream at the free; nullptr when the freeing thread had synchronised
};
struct Pool {
    std::mutex mu;
    std::multimap<size_t, FreeBlock> free_blocks;  // rounded size -> block
    std::unordered_map<void*, size_t> live;        // handed-out block -> rounded size
    std::vector<cudaEvent_t> spare_events;         // events of reused blocks, recycled
    size_t held = 0;                               // bytes obtained from the driver
};
Pool g_pools[16];
size_t g_alloc_limit = 0;

size_t round_size(size_t bytes) {
    if (bytes < 256) bytes = 256;
    if (bytes >= (size_t(1) << 20)) {
        const size_t g = size_t(2) << 20;
        return (bytes + g - 1) / g * g;
    }
    size_t r = 256;
    while (r < bytes) r <<= 1;
    return r;
}
}  // namespace

int set_error(int status, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(tls_error, sizeof(tls_error), fmt, ap);
    va_end(ap);
    return status;
}

int get_ctx(Ctx** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return set_error(DOCC_B200_ERR_NO_DEVICE, "no CUDA device: %s", cudaGetErrorString(e));
    }
    if (dev < 0 || dev >= 16) return set_error(DOCC_B200_ERR_NO_DEVICE, "device index %d out of range", dev);
    Ctx* c = &tls_ctx[dev];
    if (c->device != dev) {
        cudaDeviceProp prop;
        DOCC_CUDA_TRY(cudaGetDeviceProperties(&prop, dev));
        if (prop.major != 10) {
            return set_error(DOCC_B200_ERR_NO_DEVICE, "device %d is sm_%d%d; this library holds sm_100a code only", dev,
                             prop.major, prop.minor);
        }
        c->sm_count = prop.multiProcessorCount;
        c->cc_major = prop.major;
        DOCC_CUDA_TRY(cudaStreamCreateWithFlags(&c->own_stream, cudaStreamNonBlocking));
        for (auto& s : c->copy_streams) DOCC_CUDA_TRY(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
        for (auto& ev : c->copy_events) DOCC_CUDA_TRY(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
        DOCC_CUDA_TRY(cudaEventCreateWithFlags(&c->switch_event, cudaEventDisableTiming));
        void* h = nullptr;
        DOCC_CUDA_TRY(cudaHostAlloc(&h, sizeof(DeviceStatus), cudaHostAllocMapped));
        memset(h, 0, sizeof(DeviceStatus));
        c->status_host = static_cast<DeviceStatus*>(h);
        void* d = nullptr;
        DOCC_CUDA_TRY(cudaHostGetDevicePointer(&d, h, 0));
        c->status_dev = static_cast<DeviceStatus*>(d);
        c->stream = c->own_stream;
        c->device = dev;
    }
    *out = c;
    return DOCC_B200_OK;
}

namespace {
// The stream the calling thread's launches go to on device `dev` (nullptr before the thread's first call there).
cudaStream_t current_stream_of_thread(int dev) {
    const Ctx& c = tls_ctx[dev & 15];
    return c.device == dev ? c.stream : nullptr;
}
}  // namespace

int pool_alloc(void** dptr, size_t bytes) {
    int dev = 0;
    DOCC_CUDA_TRY(cudaGetDevice(&dev));
    Pool& p = g_pools[dev & 15];
    const size_t r = round_size(bytes);
    const cudaStream_t stream = current_stream_of_thread(dev);
    {
        std::unique_lock<std::mutex> lock(p.mu);
        auto range = p.free_blocks.equal_range(r);
        auto pick = range.second;
        for (auto it = range.first; it != range.second; ++it) {  // same stream first: no wait at all
            if (it->second.event == nullptr || it->second.stream == stream) {
                pick = it;
                break;
            }
            if (pick == range.second) pick = it;
        }
        if (pick != range.second) {
            FreeBlock b = pick->second;
            p.free_blocks.erase(pick);
            p.live[b.ptr] = r;
            lock.unlock();
            if (b.event) {
                cudaError_t e = cudaSuccess;
                if (b.stream != stream) {
                    // the block's last use was queued on another stream: order this thread's stream after it
                    e = stream ? cudaStreamWaitEvent(stream, b.event, 0) : cudaEventSynchronize(b.event);
                }
                std::lock_guard<std::mutex> relock(p.mu);
                p.spare_events.push_back(b.event);
                if (e != cudaSuccess) {
                    (void)cudaGetLastError();
                    p.free_blocks.emplace(r, FreeBlock{b.ptr, nullptr, nullptr});
                    p.live.erase(b.ptr);
                    return set_error(DOCC_B200_ERR_CUDA, "ordering a reused block after its previous owner failed: %s",
                                     cudaGetErrorString(e));
                }
            }
            *dptr = b.ptr;
            return DOCC_B200_OK;
        }
        if (g_alloc_limit && p.held + r > g_alloc_limit) {
            return set_error(DOCC_B200_ERR_OOM, "allocation of %zu bytes exceeds the configured limit of %zu (held %zu)", r,
                             g_alloc_limit, p.held);
        }
    }
    void* d = nullptr;
    cudaError_t e = cudaMalloc(&d, r);
    if (e == cudaErrorMemoryAllocation) {
        // give cached blocks back to the driver and retry once
        (void)cudaGetLastError();
        std::vector<void*> to_free;
        {
            std::lock_guard<std::mutex> lock(p.mu);
            for (auto& kv : p.free_blocks) {
                to_free.push_back(kv.second.ptr);
                if (kv.second.event) p.spare_events.push_back(kv.second.event);
                p.held -= kv.first;
            }
            p.free_blocks.clear();
        }
        (void)cudaDeviceSynchronize();
        for (void* q : to_free) (void)cudaFree(q);
        e = cudaMalloc(&d, r);
    }
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return set_error(e == cudaErrorMemoryAllocation ? DOCC_B200_ERR_OOM : DOCC_B200_ERR_CUDA, "cudaMalloc(%zu): %s", r,
                         cudaGetErrorString(e));
    }
    std::lock_guard<std::mutex> lock(p.mu);
    p.held += r;
    p.live[d] = r;
    *dptr = d;
    return DOCC_B200_OK;
}

int pool_free(void* dptr) {
    if (!dptr) return DOCC_B200_OK;
    int dev = 0;
    DOCC_CUDA_TRY(cudaGetDevice(&dev));
    Pool& p = g_pools[dev & 15];
    const cudaStream_t stream = current_stream_of_thread(dev);
    cudaEvent_t ev = nullptr;
    size_t r = 0;
    {
        std::lock_guard<std::mutex> lock(p.mu);
        auto it = p.live.find(dptr);
        if (it == p.live.end()) return set_error(DOCC_B200_ERR_INVALID_ARG, "pointer %p was not allocated by docc_b200_malloc", dptr);
        r = it->second;
        p.live.erase(it);
        if (!p.spare_events.empty()) {
            ev = p.spare_events.back();
            p.spare_events.pop_back();
        }
    }
    // Mark the point on the freeing thread's stream after which the block is no longer in use. If that cannot be done
    // (no stream yet, or the event calls fail) the free falls back to waiting for the device, which is always safe.
    bool marked = false;
    if (stream) {
        if (!ev && cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess) ev = nullptr;
        if (ev && cudaEventRecord(ev, stream) == cudaSuccess) marked = true;
    }
    if (!marked) {
        (void)cudaGetLastError();
        (void)cudaDeviceSynchronize();
    }
    std::lock_guard<std::mutex> lock(p.mu);
    if (!marked && ev) {
        p.spare_events.push_back(ev);
        ev = nullptr;
    }
    p.free_blocks.emplace(r, FreeBlock{dptr, stream, ev});
    return DOCC_B200_OK;
}

int get_workspace(Ctx* ctx, int slot, size_t bytes, void** out) {
    if (ctx->workspace_bytes[slot] < bytes) {
        if (ctx->workspace[slot]) {
            // other work queued on the stream may still read the old block
            DOCC_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
            DOCC_TRY(pool_free(ctx->workspace[slot]));
            ctx->workspace[slot] = nullptr;
            ctx->workspace_bytes[slot] = 0;
        }
        DOCC_TRY(pool_alloc(&ctx->workspace[slot], bytes));
        ctx->workspace_bytes[slot] = round_size(bytes);
    }
    *out = ctx->workspace[slot];
    return DOCC_B200_OK;
}

int after_launch(Ctx* ctx, const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return set_error(DOCC_B200_ERR_CUDA, "launch of %s failed: %s", what, cudaGetErrorString(e));
    ctx->launches++;
    return DOCC_B200_OK;
}

}  // namespace docc_b200

using namespace docc_b200;

extern "C" {

int docc_b200_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        (void)cudaGetLastError();
        return 0;
    }
    return n;
}

int docc_b200_init(int device) {
    int n = docc_b200_device_count();
    if (n == 0) return set_error(DOCC_B200_ERR_NO_DEVICE, "no CUDA device is visible");
    if (device < 0 || device >= n) return set_error(DOCC_B200_ERR_INVALID_ARG, "device %d out of range [0,%d)", device, n);
    DOCC_CUDA_TRY(cudaSetDevice(device));
    Ctx* c;
    return get_ctx(&c);
}

int docc_b200_shutdown(void) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) {
        (void)cudaGetLastError();
        return DOCC_B200_OK;
    }
    Ctx* c = &tls_ctx[dev & 15];
    if (c->device != dev) return DOCC_B200_OK;
    DOCC_CUDA_TRY(cudaStreamSynchronize(c->stream));
    for (int i = 0; i < 4; i++) {
        if (c->workspace[i]) pool_free(c->workspace[i]);
        c->workspace[i] = nullptr;
        c->workspace_bytes[i] = 0;
    }
    Pool& p = g_pools[dev & 15];
    std::vector<void*> to_free;
    {
        std::lock_guard<std::mutex> lock(p.mu);
        for (auto& kv : p.free_blocks) {
            to_free.push_back(kv.second.ptr);
            if (kv.second.event) p.spare_events.push_back(kv.second.event);
            p.held -= kv.first;
        }
        p.free_blocks.clear();
    }
    (void)cudaDeviceSynchronize();  // blocks freed on other threads' streams may still be in use there
    for (void* q : to_free) (void)cudaFree(q);
    return DOCC_B200_OK;
}

int docc_b200_malloc(void** dptr, size_t bytes) {
    DOCC_REQUIRE(dptr != nullptr, "docc_b200_malloc: dptr is NULL");
    Ctx* c;
    DOCC_TRY(get_ctx(&c));
    return pool_alloc(dptr, bytes);
}

int docc_b200_free(void* dptr) {
    if (!dptr) return DOCC_B200_OK;
    Ctx* c;
    DOCC_TRY(get_ctx(&c));
    // asynchronous: the pool orders the block's next owner after the work queued on this thread's stream so far
    return pool_free(dptr);
}

int docc_b200_h2d(void* dptr, const void* hptr, size_t bytes) {
    DOCC_REQUIRE(bytes == 0 || (dptr && hptr), "docc_b200_h2d: NULL pointer");
    Ctx* c;
    DOCC_TRY(get_ctx(&c));
    if (bytes == 0) return DOCC_B200_OK;
    DOCC_CUDA_TRY(cudaMemcpyAsync(dptr, hptr, bytes, cudaMemcpyHostToDevice, c->stream));
    DOCC_CUDA_TRY(cudaStreamSynchronize(c->stream));
    return DOCC_B200_OK;
}

int docc_b200_d2h(void* hptr, const void* dptr, size_t bytes) {
    DOCC_REQUIRE(bytes == 0 || (dptr && hptr), "docc_b200_d2h: NULL pointer");
    Ctx* c;
    DOCC_TRY(get_ctx(&c));
    if (bytes == 0) return DOCC_B200_OK;
    DOCC_CUDA_TRY(cudaMemcpyAsync(hptr, dptr, bytes, cudaMemcpyDeviceToHost, c->stream));
    DOCC_CUDA_TRY(cudaStreamSynchronize(c->stream));
    return DOCC_B200_OK;
}

int docc_b200_host_alloc(void** hptr, size_t bytes) {
    DOCC_REQUIRE(hptr != nullptr, "docc_b200_host_alloc: hptr is NULL");
    Ctx* c;
    DOCC_TRY(get_ctx(&c));
    DOCC_CUDA_TRY(cudaHostAlloc(hptr, bytes ? bytes : 1, cudaHostAllocDefault));
    return DOCC_B200_OK;
}

int docc_b200_host_free(void* hptr) {
    if (!hptr) return DOCC_B200_OK;
    DOCC_CUDA_TRY(cudaFreeHost(hptr));
    return DOCC_B200_OK;
}

int docc_b200_set_alloc_limit(size_t bytes) {
    g_alloc_limit = bytes;
    return DOCC_B200_OK;
}

int docc_b200_set_stream(void* stream) {
    Ctx* c;
    DOCC_TRY(get_ctx(&c));
    const cudaStream_t next = stream ? static_cast<cudaStream_t>(stream) : c->own_stream;
    if (next != c->stream) {
        // The thread's workspaces (operand planes, block intermediates) and the buffers it handed out are ordered on
        // one stream at a time. Work already queued on the old stream may still use them, so the new stream is made
        // to wait for it; the host does not block.
        cudaEvent_t ev = c->switch_event;
        cudaError_t e = cudaEventRecord(ev, c->stream);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(next, ev, 0);
        const cudaStream_t old = c->stream;
        c->stream = next;  // the switch itself always takes effect
        if (e != cudaSuccess) {
            (void)cudaGetLastError();
            (void)old;
            DOCC_CUDA_TRY(cudaDeviceSynchronize());  // e.g. the old stream handle was destroyed by its owner
        }
    }
    return DOCC_B200_OK;
}

int docc_b200_get_stream(void** stream) {
    DOCC_REQUIRE(stream != nullptr, "docc_b200_get_stream: stream is NULL");
    Ctx* c;
    DOCC_TRY(get_ctx(&c));
    *stream = c->stream;
    return DOCC_B200_OK;
}

int docc_b200_sync(void) {
    Ctx* c;
    DOCC_TRY(get_ctx(&c));
    DOCC_CUDA_TRY(cudaStreamSynchronize(c->stream));
    if (c->status_host->timeout_flag) {
        unsigned where = c->status_host->timeout_where;
        c->status_host->timeout_flag = 0;
        c->status_host->timeout_where = 0;
        return set_error(DOCC_B200_ERR_DEVICE_TIMEOUT, "a bounded device-side wait ran out (location code %u)", where);
    }
    return DOCC_B200_OK;
}

const char* docc_b200_strerror(int status) {
    switch (status) {
        case DOCC_B200_OK: return "ok";
        case DOCC_B200_ERR_INVALID_ARG: return "invalid argument";
        case DOCC_B200_ERR_UNSUPPORTED: return "unsupported configuration";
        case DOCC_B200_ERR_CUDA: return "CUDA call failed";
        case DOCC_B200_ERR_OOM: return "out of memory";
        case DOCC_B200_ERR_NO_DEVICE: return "no usable sm_100 device";
        case DOCC_B200_ERR_DEVICE_TIMEOUT: return "device-side wait timed out";
        default: return "unknown status";
    }
}

const char* docc_b200_last_error(void) { return tls_error; }

int64_t docc_b200_launch_count(int reset) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) {
        (void)cudaGetLastError();
        return 0;
    }
    Ctx* c = &tls_ctx[dev & 15];
    int64_t v = c->launches;
    if (reset) c->launches = 0;
    return v;
}

}  // extern "C"
