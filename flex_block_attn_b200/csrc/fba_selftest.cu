// Self-test of the bounded-wait path: the one place where a wait is MEANT to run out.
//
// Every spin in the attention kernels goes through mbar_wait(), which gives up after a cycle budget,
// raises the CTA's abort flag and lets the role record where it stopped in the caller's status
// words.  In a correct run that path never executes, so this file exercises it on a toy: one CTA
// initialises an mbarrier that nobody ever arrives at, one thread waits on it with a short budget,
// the wait returns false by itself, the thread records (kernel 9, role 1, tag 777) and the kernel
// ends normally.  Nothing traps, faults or spins without a limit; the context stays usable.
#include "fba_common.cuh"

namespace fba {

__global__ void __launch_bounds__(64) selftest_wait_kernel(uint32_t* status, long long limit_cycles,
                                                           unsigned long long* waited_cycles) {
    __shared__ __align__(8) unsigned long long bar_storage;
    __shared__ int abort_word;
    volatile int* abort_flag = &abort_word;
    const uint32_t bar = smem_u32(&bar_storage);
    if (threadIdx.x == 0) {
        *abort_flag = 0;
        mbar_init(bar, 1);
        mbar_fence_init();
    }
    __syncthreads();
    if (threadIdx.x == 32) {
        const long long t0 = clock64();
        const bool ok = mbar_wait(bar, 0, abort_flag, limit_cycles);   // phase 0 never completes
        if (waited_cycles) *waited_cycles = static_cast<unsigned long long>(clock64() - t0);
        if (!ok) report_timeout(status, 9, 1, 0, 777);
    }
    __syncthreads();
    // Every other thread sees the abort flag the waiter raised, exactly as the roles of the
    // attention kernels do before they fall through to their common exit.
    if (threadIdx.x == 0 && *abort_flag != 1) report_timeout(status, 9, 2, 0, 778);
}

}  // namespace fba

using namespace fba;

extern "C" int fba_selftest_wait_timeout(uint32_t* status, int64_t limit_cycles, uint64_t* waited_cycles,
                                         void* stream) {
    if (!status) return set_error(FBA_ERR_BAD_ARG, "fba_selftest_wait_timeout: null status buffer");
    if (limit_cycles <= 0 || limit_cycles > 2000000000LL)
        return set_error(FBA_ERR_BAD_ARG, "fba_selftest_wait_timeout: limit must be in (0, 2e9] cycles");
    DeviceGuard guard;
    int rc = guard.bind(status);
    if (rc != FBA_OK) return rc;
    selftest_wait_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(
        status, static_cast<long long>(limit_cycles), reinterpret_cast<unsigned long long*>(waited_cycles));
    return check_launch("selftest_wait_kernel");
}
