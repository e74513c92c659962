// Self-test of the bounded-wait convention the pipelined kernels share: every wait on an mbarrier polls a limited
// number of times, raises the block's abort flag, and the kernel reports status 3 and returns instead of hanging.
// The kernel below waits on a barrier that nothing ever arrives at, so the limit is what ends it.
#include "common.cuh"
#include "tc_common.cuh"

namespace {

__global__ void bounded_wait_selftest_kernel(int32_t* status, uint32_t limit) {
    __shared__ uint64_t bar;
    __shared__ volatile int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        tc::mbar_init(&bar, 1);
        tc::mbar_init_fence();
    }
    __syncthreads();
    const bool ok = tc::mbar_wait(&bar, 0, &abort_flag, limit);   // phase 0 never completes: no arrival is ever made
    __syncthreads();
    if (threadIdx.x == 0 && (!ok || abort_flag)) atomicExch(status, 3);
}

}  // namespace

extern "C" int e3b_selftest_bounded_wait(int32_t* status, unsigned limit, void* stream) {
    if (!status) return e3b::fail(E3B_ERR_ARG, "e3b_selftest_bounded_wait: null status pointer");
    if (limit == 0 || limit > 100000u) return e3b::fail(E3B_ERR_ARG, "e3b_selftest_bounded_wait: limit must be in [1, 100000]");
    bounded_wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(status, limit);
    return e3b::check_launch("bounded_wait_selftest_kernel");
}
