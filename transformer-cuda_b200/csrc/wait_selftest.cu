// Self-test of the bounded waits: a one-CTA kernel waits on an mbarrier that nothing ever arrives on, with a
// limit of a few thousand polls instead of the production limit, so that the whole error chain can be
// exercised on a healthy GPU in well under a second: the wait gives up, sets the CTA's abort flag, records
// kFaultWaitTimeout | id in the device fault word, a second wait returns early because of the flag, and the
// kernel runs to its normal end. Nothing traps, faults or spins without a limit.
#include "kernels.cuh"
#include "tc_common.cuh"

namespace b200attn {
namespace {

constexpr uint32_t kSelfTestPolls = 4096;

__global__ void __launch_bounds__(64) wait_selftest_kernel(unsigned int* fault_word, unsigned int* report) {
    __shared__ uint64_t never_signalled;
    __shared__ uint32_t abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(&never_signalled, 1);
        abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) mbar_wait_limited(&never_signalled, 0, &abort_flag, fault_word, kWaitSelfTestId, kSelfTestPolls);
    __syncthreads();
    // with the flag set, a wait that would otherwise poll a million times leaves after its first 1024 polls
    long long t0 = clock64();
    if (threadIdx.x == 32) mbar_wait_limited(&never_signalled, 0, &abort_flag, nullptr, kWaitSelfTestId + 1, 1u << 20);
    long long t1 = clock64();
    __syncthreads();
    if (threadIdx.x == 32 && report) {
        report[0] = abort_flag;
        report[1] = (unsigned int)((t1 - t0) >> 10);  // cycles / 1024 the second wait took
    }
}

}  // namespace

cudaError_t launch_wait_selftest(unsigned int* fault_word, unsigned int* report, cudaStream_t stream) {
    wait_selftest_kernel<<<1, 64, 0, stream>>>(fault_word, report);
    return cudaGetLastError();
}

}  // namespace b200attn
