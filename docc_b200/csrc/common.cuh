// Shared host-side plumbing of the docc_b200 runtime: per-thread context, error
// reporting, pooled device memory, workspaces and launch accounting.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <utility>

#include "docc_b200/rt.h"

namespace docc_b200 {

// ---- error reporting -----------------------------------------------------------------
int set_error(int status, const char* fmt, ...);

#define DOCC_CUDA_TRY(expr)                                                                              \
    do {                                                                                                 \
        cudaError_t _e = (expr);                                                                         \
        if (_e != cudaSuccess) {                                                                         \
            (void)cudaGetLastError();                                                                    \
            return ::docc_b200::set_error(_e == cudaErrorMemoryAllocation ? DOCC_B200_ERR_OOM            \
                                                                          : DOCC_B200_ERR_CUDA,          \
                                          "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e),        \
                                          __FILE__, __LINE__);                                           \
        }                                                                                                \
    } while (0)

#define DOCC_TRY(expr)                   \
    do {                                 \
        int _s = (expr);                 \
        if (_s != DOCC_B200_OK) return _s; \
    } while (0)

#define DOCC_REQUIRE(cond, ...)                                                   \
    do {                                                                          \
        if (!(cond)) return ::docc_b200::set_error(DOCC_B200_ERR_INVALID_ARG, __VA_ARGS__); \
    } while (0)

// ---- context ----------------------------------------------------------------------------
// Word 0 of the status block is written by kernels whose bounded waits run out; it lives in
// mapped pinned host memory so the host can read it after a sync without a copy.
struct DeviceStatus {
    unsigned int timeout_flag;   // != 0: a bounded device-side wait expired
    unsigned int timeout_where;  // kernel-specific location code
    unsigned int pad[14];
};

struct Ctx {
    int device = -1;
    cudaStream_t own_stream = nullptr;  // created lazily, non-blocking
    cudaStream_t stream = nullptr;      // the stream launches go to (own_stream unless overridden)
    cudaStream_t copy_streams[2] = {nullptr, nullptr};
    cudaEvent_t copy_events[4] = {nullptr, nullptr, nullptr, nullptr};
    cudaEvent_t switch_event = nullptr;  // orders a newly selected stream after the one it replaces
    void* workspace[4] = {nullptr, nullptr, nullptr, nullptr};  // library-owned scratch, grows on demand
    size_t workspace_bytes[4] = {0, 0, 0, 0};
    DeviceStatus* status_host = nullptr;  // mapped pinned
    DeviceStatus* status_dev = nullptr;   // device alias of status_host
    int sm_count = 0;
    int cc_major = 0;
    int64_t launches = 0;
};

// Returns the calling thread's context for the current device (creating it on first use).
int get_ctx(Ctx** out);
// Library-owned scratch slot `slot` of at least `bytes` bytes (contents undefined).
int get_workspace(Ctx* ctx, int slot, size_t bytes, void** out);
// Checks cudaGetLastError after a launch and counts it.
int after_launch(Ctx* ctx, const char* what);
// Pool interface (also behind docc_b200_malloc / docc_b200_free).
int pool_alloc(void** dptr, size_t bytes);
int pool_free(void* dptr);

inline size_t prec_size(int prec) {
    switch (prec) {
        case DOCC_B200_PREC_D: return 8;
        case DOCC_B200_PREC_S: return 4;
        case DOCC_B200_PREC_H:
        case DOCC_B200_PREC_B: return 2;
        default: return 0;
    }
}

// RAII set of temporary device buffers used by the host-pointer ("WithTransfers") variants.
struct TempBuffers {
    void* ptrs[8];
    int n = 0;
    ~TempBuffers() {
        for (int i = 0; i < n; i++) pool_free(ptrs[i]);
    }
    int alloc(void** out, size_t bytes) {
        int s = pool_alloc(out, bytes ? bytes : 1);
        if (s == DOCC_B200_OK) ptrs[n++] = *out;
        return s;
    }
};

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Launch with programmatic stream serialization: the kernel may become resident while the kernel before it in the
// stream is still running, so its launch latency and set-up (barrier initialisation, tensor-memory allocation,
// descriptor prefetch) disappear behind that kernel's tail. Only for kernels that execute griddepcontrol.wait
// (ptx::griddep_wait) before their first access to global memory; the wait returns once the earlier kernel has
// completed and its writes are visible, so no data dependence is relaxed.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

}  // namespace docc_b200
