// Self-test of the bounded-wait machinery the tensor-core kernels rely on, in a form that cannot hurt a device:
// a tiny kernel with the same roles in miniature. One role waits on an mbarrier nobody ever arrives on, with a
// caller-chosen (short) limit; it gives up through mbar_wait_limit (the very function the kernels' waits go
// through), raises the abort flag and records a code in the status word. A second role waits on another barrier
// with the kernels' ordinary limit and must leave early because it sees the flag. The CTA then releases the tensor
// memory it holds and returns: no trap, no assert, no spinning beyond the limit. The host reads the status word and
// reports it exactly as Model::forward does.
#include <cuda_runtime.h>

#include "common.cuh"
#include "kernels.hpp"
#include "pool.hpp"
#include "ptx_sm100.cuh"

namespace bfb {

namespace {

__global__ void __launch_bounds__(96, 1) boundedWaitSelfTestKernel(unsigned long long limitNs, int* status, int* observed) {
    __shared__ uint64_t neverArrives;
    __shared__ uint64_t alsoNever;
    __shared__ uint32_t tmemSlot;
    __shared__ int abortFlag;
    const int warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        mbar_init(&neverArrives, 1);
        mbar_init(&alsoNever, 1);
        abortFlag = 0;
        fence_mbar_init();
    }
    if (warp == 0) {
        tmem_alloc(&tmemSlot, 32);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmemBase = tmemSlot;
    volatile int* abortPtr = &abortFlag;
    if (warp == 1) {
        // the wait that runs out
        const bool ok = warp_all(mbar_wait_limit(&neverArrives, 0u, abortPtr, status, kDevTimeoutOther, limitNs));
        if (threadIdx.x == 32) observed[0] = ok ? 1 : 0;
    } else if (warp == 2) {
        // a role with the ordinary limit: it must leave because of the flag, long before its own limit
        const unsigned long long t0 = global_timer_ns();
        const bool ok = warp_all(mbar_wait(&alsoNever, 0u, abortPtr, status, kDevTimeoutAccFull));
        if (threadIdx.x == 64) {
            observed[1] = ok ? 1 : 0;
            observed[2] = static_cast<int>(min(global_timer_ns() - t0, 2000000000ull) / 1000ull);   // microseconds
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmemBase, 32);
    }
}

}  // namespace

// Runs the self-test on `stream` with the given limit for the wait that must run out. Returns the device status
// code (0 when the wait did not expire, which cannot happen); `observedHost` receives {first wait succeeded,
// second wait succeeded, microseconds the second role waited}.
int selfTestBoundedWait(unsigned long long limitNs, int* observedHost, cudaStream_t stream) {
    require(limitNs >= 1000ull && limitNs <= 1000000000ull, "selftest_bounded_wait: limit must be 1 us .. 1 s");
    int* d = static_cast<int*>(poolAcquire(4 * sizeof(int)));
    int host[4] = {0, 0, 0, 0};
    try {
        BFB_CUDA(cudaMemsetAsync(d, 0, 4 * sizeof(int), stream));
        boundedWaitSelfTestKernel<<<1, 96, 0, stream>>>(limitNs, d, d + 1);
        BFB_LAUNCH_CHECK();
        noteLaunch();
        BFB_CUDA(cudaMemcpyAsync(host, d, sizeof(host), cudaMemcpyDeviceToHost, stream));
        BFB_CUDA(cudaStreamSynchronize(stream));
    } catch (...) {
        poolRelease(d, 4 * sizeof(int));
        throw;
    }
    poolRelease(d, 4 * sizeof(int));
    if (observedHost != nullptr) {
        observedHost[0] = host[1];
        observedHost[1] = host[2];
        observedHost[2] = host[3];
    }
    return host[0];
}

}  // namespace bfb
