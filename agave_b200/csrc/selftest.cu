// A unit kernel for the give-up path of the bounded waits.
//
// The tensor-core kernels wait on mbarriers with tc5::mbar_wait, which polls a bounded
// number of times and then returns false; the kernel that called it records a code in a
// status word, stops issuing work, frees its tensor memory and returns, so that the
// context stays usable.  In a healthy run no wait ever gives up, so that path would never
// execute.  This kernel executes it on purpose and harmlessly: it follows the same
// protocol as the product kernels (barriers initialised by one thread, tensor memory
// allocated by warp 1, a loader that waits for a free stage, an issuer that watches the
// abort flag, an epilogue that waits for the accumulator), but nothing ever arrives on
// its barriers and every wait gets a limit of a few thousand polls.  Nothing traps,
// nothing spins without a bound.  The reference has no counterpart (it has no
// asynchronous barriers to wait on).
#include "common.cuh"
#include "tcgen05.cuh"

using namespace tc5;

namespace {

__global__ void __launch_bounds__(192, 1)
bounded_wait_selftest_kernel(unsigned limit, int* __restrict__ status, unsigned* __restrict__ polls) {
    __shared__ __align__(8) uint64_t empty_bar, acc_full;
    __shared__ uint32_t tmem_slot;
    __shared__ volatile int abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        mbar_init(&empty_bar, 1);
        mbar_init(&acc_full, 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(&tmem_slot)),
                     "r"(32u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    if (warp == 0 && lane == 0) {
        // loader: a fresh barrier is in phase 0, so a wait for parity 0 never returns
        // true unless somebody arrives, and nobody does
        const long long t0 = clock64();
        if (!mbar_wait(&empty_bar, 0, limit)) {
            atomicCAS(status, 0, (1 << 8) | 0);
            abort_flag = 1;
        }
        polls[0] = (unsigned)(clock64() - t0);
    } else if (warp == 1 && lane == 0) {
        // issuer: gives up when the abort flag is up (bounded by the loader's limit)
        for (unsigned i = 0; i < 64u * limit && !abort_flag; ++i) __nanosleep(20);
    } else if (warp >= 2) {
        // epilogue: waits for an accumulator that never comes
        if (!mbar_wait(&acc_full, 0, limit)) {
            atomicCAS(status, 0, (3 << 8));
            abort_flag = 1;
        }
    }
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"(32u)
                     : "memory");
    }
}

}  // namespace

// Runs the kernel above on `ctas` CTAs with every wait limited to `limit` polls
// (1..65536).  status (one int on the device, zero before) receives the code of the
// first wait that gave up: (1 << 8) for the loader, (3 << 8) for the epilogue.
// cycles (one unsigned per call) receives the clock cycles the loader's wait took.
AGV_API int agv_selftest_bounded_wait(unsigned limit, int ctas, int* status, unsigned* cycles,
                                      cudaStream_t stream) {
    AGV_REQUIRE(limit >= 1 && limit <= 65536, "selftest: the limit must be 1..65536 polls");
    AGV_REQUIRE(ctas >= 1 && ctas <= 1024, "selftest: 1..1024 CTAs");
    AGV_REQUIRE(status && cycles, "selftest: null pointers");
    agv_launch(bounded_wait_selftest_kernel, dim3(ctas), dim3(192), 0, stream, limit, status, cycles);
    AGV_LAUNCH_OK("bounded_wait_selftest_kernel");
    return 0;
}
