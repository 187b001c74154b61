// docc_b200_gemm_f32_noalloc: the fp32 tensor-core GEMM for callers that must not allocate.
//
// The regular fp32 GEMM (docc_b200_gemm, precision 's') splits A and B into bf16 hi/lo planes in a
// pooled workspace that grows through cudaMalloc, and its first call on a thread creates streams and
// a pinned status word. Some embedders cannot accept any of that: a host application that handed
// the whole device to its own allocator at start-up leaves nothing for a later cudaMalloc, and a
// latency-critical loop cannot take the device-wide synchronisation a cudaMalloc / cudaFree implies.
// This entry point therefore works out of one fixed array that is part of the library image:
// the planes live in `g_noalloc_scratch` below, the caller supplies the stream, and no
// allocating call of the CUDA runtime, the driver or any framework is made.
//
// Cost and limits: every GPU that loads this library holds kNoAllocScratchBytes (16 MiB) until
// the process exits. A call needs 4 * (m + n) * roundup8(k) bytes of it; larger problems are
// rejected with DOCC_B200_ERR_INVALID_ARG. All calls share the array and it keeps the previous
// call's planes, so two calls that overlap on the GPU (different streams, or different host
// threads) race on it — serialise them. Nothing in the array has to start at zero (every plane
// element a call reads is written by that call first); the kernel status word is cleared on every call.
//
// The first call on a device resolves the device address of the array (cudaGetSymbolAddress) and
// sets the kernel's shared-memory attribute; make that first call outside any stream capture.
// The call returns after the product is complete on `stream`.
#include <mutex>

#include "gemm_tc.h"

namespace docc_b200 {
namespace {

constexpr size_t kNoAllocScratchBytes = size_t(16) << 20;

// In host code these names are only handles for cudaGetSymbolAddress / cudaMemcpyFromSymbol; the
// device addresses are resolved once per device in setup() and passed to the kernels as pointers.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];
static __device__ __align__(256) DeviceStatus g_noalloc_status;

struct PerDevice {
    bool ready = false;
    void* scratch = nullptr;
    DeviceStatus* status = nullptr;
    int sm_count = 0;
};
PerDevice g_dev[16];
std::mutex g_setup_mu;

int setup(int dev, PerDevice** out) {
    std::lock_guard<std::mutex> lock(g_setup_mu);
    PerDevice& d = g_dev[dev];
    if (!d.ready) {
        int major = 0;
        DOCC_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
        if (major != 10) return set_error(DOCC_B200_ERR_NO_DEVICE, "device %d is not sm_100", dev);
        DOCC_CUDA_TRY(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev));
        void* p = nullptr;
        DOCC_CUDA_TRY(cudaGetSymbolAddress(&p, g_noalloc_scratch));
        d.scratch = p;
        void* s = nullptr;
        DOCC_CUDA_TRY(cudaGetSymbolAddress(&s, g_noalloc_status));
        d.status = static_cast<DeviceStatus*>(s);
        d.ready = true;
    }
    *out = &d;
    return DOCC_B200_OK;
}

int64_t round_up8(int64_t v) { return (v + 7) / 8 * 8; }

}  // namespace
}  // namespace docc_b200

using namespace docc_b200;

extern "C" int docc_b200_gemm_f32_noalloc(int transa, int transb, int64_t m, int64_t n, int64_t k, float alpha, const float* A,
                                          int64_t lda, const float* B, int64_t ldb, float beta, float* C, int64_t ldc,
                                          void* stream) {
    DOCC_REQUIRE(transa == DOCC_B200_NO_TRANS || transa == DOCC_B200_TRANS, "gemm_f32_noalloc: unknown transA %d", transa);
    DOCC_REQUIRE(transb == DOCC_B200_NO_TRANS || transb == DOCC_B200_TRANS, "gemm_f32_noalloc: unknown transB %d", transb);
    DOCC_REQUIRE(m >= 0 && n >= 0 && k >= 1, "gemm_f32_noalloc: m, n must be >= 0 and k >= 1");
    if (m == 0 || n == 0) return DOCC_B200_OK;
    DOCC_REQUIRE(A && B && C, "gemm_f32_noalloc: NULL matrix pointer");
    const bool ta = transa == DOCC_B200_TRANS, tb = transb == DOCC_B200_TRANS;
    DOCC_REQUIRE(lda >= (ta ? m : k) && ldb >= (tb ? k : n) && ldc >= n, "gemm_f32_noalloc: leading dimension too small");
    // extents of a problem that fits are far below 2^31; checking first keeps the size product from wrapping
    DOCC_REQUIRE(m <= INT32_MAX && n <= INT32_MAX && k <= INT32_MAX - 8, "gemm_f32_noalloc: extent exceeds 2^31 - 1");
    const int64_t kp = round_up8(k);
    // hi + lo planes of A and of B, 2 bytes each. The comparison divides so that no product can wrap; `need` is only
    // formed for the message when it is known to be huge, where saturating is good enough.
    const bool too_big = uint64_t(m + n) > kNoAllocScratchBytes / 4 / uint64_t(kp);
    const size_t need = too_big && uint64_t(m + n) > (UINT64_MAX / 4) / uint64_t(kp) ? SIZE_MAX
                                                                                     : size_t(4) * size_t(m + n) * size_t(kp);
    if (too_big) {
        return set_error(DOCC_B200_ERR_INVALID_ARG,
                         "gemm_f32_noalloc: problem needs %zu bytes of scratch (4*(m+n)*roundup8(k)) but the built-in array holds "
                         "%zu; use docc_b200_gemm for larger products",
                         need, kNoAllocScratchBytes);
    }
    int dev = 0;
    DOCC_CUDA_TRY(cudaGetDevice(&dev));
    DOCC_REQUIRE(dev >= 0 && dev < 16, "gemm_f32_noalloc: device index out of range");
    PerDevice* d;
    DOCC_TRY(setup(dev, &d));

    // A context on the stack: the caller's stream, the static status word, nothing owned.
    Ctx ctx;
    ctx.device = dev;
    ctx.stream = static_cast<cudaStream_t>(stream);
    ctx.sm_count = d->sm_count;
    ctx.cc_major = 10;
    ctx.status_dev = d->status;

    DOCC_CUDA_TRY(cudaMemsetAsync(d->status, 0, sizeof(DeviceStatus), ctx.stream));
    __nv_bfloat16* a_hi = static_cast<__nv_bfloat16*>(d->scratch);
    __nv_bfloat16* a_lo = a_hi + size_t(m) * kp;
    __nv_bfloat16* b_hi = a_lo + size_t(m) * kp;
    __nv_bfloat16* b_lo = b_hi + size_t(n) * kp;
    // planes are K-major: A as [m][kp], B as [n][kp]; the split transposes when the source is not
    if (!ta) DOCC_TRY(split_f32_to_bf16x2(&ctx, A, m, k, lda, 1, 0, false, a_hi, a_lo, kp, 0));
    else DOCC_TRY(split_f32_to_bf16x2(&ctx, A, k, m, lda, 1, 0, true, a_hi, a_lo, kp, 0));
    if (tb) DOCC_TRY(split_f32_to_bf16x2(&ctx, B, n, k, ldb, 1, 0, false, b_hi, b_lo, kp, 0));
    else DOCC_TRY(split_f32_to_bf16x2(&ctx, B, k, n, ldb, 1, 0, true, b_hi, b_lo, kp, 0));

    TcOperand a[2], b[2];
    a[0].ptr = a_hi; a[1].ptr = a_lo; b[0].ptr = b_hi; b[1].ptr = b_lo;
    for (int i = 0; i < 2; i++) {
        a[i].ld = kp; a[i].batch_stride = 0; a[i].k_major = true;
        b[i].ld = kp; b[i].batch_stride = 0; b[i].k_major = true;
    }
    TcEpilogue ep;
    ep.alpha = alpha; ep.beta = beta;
    ep.out = C; ep.ldo = ldc; ep.out_prec = DOCC_B200_PREC_S;
    const int pa[3] = {1, 0, 0}, pb[3] = {0, 1, 0};  // lo*hi, hi*lo, hi*hi — the order docc_b200_gemm uses
    DOCC_TRY(tc_gemm(&ctx, 1, m, n, k, 1, 3, a, pa, b, pb, ep));

    DeviceStatus st;
    DOCC_CUDA_TRY(cudaMemcpyAsync(&st, d->status, sizeof(st), cudaMemcpyDeviceToHost, ctx.stream));
    DOCC_CUDA_TRY(cudaStreamSynchronize(ctx.stream));
    if (st.timeout_flag)
        return set_error(DOCC_B200_ERR_DEVICE_TIMEOUT, "gemm_f32_noalloc: a bounded device-side wait ran out (location code %u)",
                         st.timeout_where);
    return DOCC_B200_OK;
}
