// Self-test entry of the bounded-wait error path.
//
// Every spin in the tensor-core kernels goes through ptx::mbar_wait, which gives up after a cycle budget; the kernel
// then writes the status word in mapped host memory, releases what it holds and returns, and the next docc_b200_sync
// reports DOCC_B200_ERR_DEVICE_TIMEOUT. In a correct run no wait ever expires, so that path would never execute.
// docc_b200_selftest_wait_timeout makes it execute harmlessly: one warp waits on an mbarrier in its own shared memory
// that nothing arrives at, with a budget the caller chooses (tests use ~10^5 clocks, about 50 microseconds). The
// kernel touches no global memory besides the status word, holds no tensor memory and has no copy in flight, so
// giving up is all the clean-up there is. The device and the context stay fully usable.
#include "common.cuh"
#include "ptx.cuh"

namespace docc_b200 {
namespace {

__global__ void __launch_bounds__(32) wait_timeout_kernel(DeviceStatus* status, long long limit_cycles, unsigned where) {
    __shared__ __align__(8) unsigned long long bar;
    const uint32_t bar_addr = ptx::smem_u32(&bar);
    if (threadIdx.x == 0) {
        ptx::mbar_init(bar_addr, 1);
        ptx::fence_barrier_init();
    }
    __syncwarp();
    // phase 0 never completes: no thread arrives and no copy is counted on this barrier
    const bool done = ptx::mbar_wait(bar_addr, 0u, limit_cycles);
    if (!done && threadIdx.x == 0) {
        volatile unsigned int* w = &status->timeout_where;
        volatile unsigned int* f = &status->timeout_flag;
        if (*w == 0u) *w = where;
        *f = 1u;
        __threadfence_system();
    }
}

}  // namespace
}  // namespace docc_b200

using namespace docc_b200;

extern "C" int docc_b200_selftest_wait_timeout(int64_t limit_cycles) {
    DOCC_REQUIRE(limit_cycles > 0 && limit_cycles <= 2000000000LL, "selftest_wait_timeout: limit must be in (0, 2e9] clocks");
    Ctx* ctx;
    DOCC_TRY(get_ctx(&ctx));
    wait_timeout_kernel<<<1, 32, 0, ctx->stream>>>(ctx->status_dev, (long long)limit_cycles, 900u);
    return after_launch(ctx, "wait_timeout_kernel");
}
