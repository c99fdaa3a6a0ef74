// A kernel for the tests of the give-up path: one CTA waits, with the same code every tensor-core
// kernel waits with, on a barrier that nobody arrives at.  The wait is bounded by a limit of a
// few thousand clock cycles given by the caller, runs out, and the kernel leaves the status word
// set and returns: nothing hangs and nothing faults.  It shows that a wait that ran out reaches
// the host (through `shiso_gemm_tcgen05_status` or with a step's picked tokens) and that the
// kernels after it run as always.
#include "tcgen05.cuh"

namespace {

__global__ void bounded_wait_kernel(unsigned long long limit_cycles, int* status) {
    __shared__ __align__(8) uint64_t barrier;
    if (threadIdx.x == 0) {
        tc::mbar_init(&barrier, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        const bool arrived = tc::mbar_wait_limit(&barrier, 0, limit_cycles);
        if (!arrived && status != nullptr) atomicExch(status, 1);
    }
}

}  // namespace

// Launches the kernel above; `limit_cycles` is clamped to 10^7 (a few milliseconds).
SHISO_API int shiso_selftest_bounded_wait(long long limit_cycles, cudaStream_t stream) {
    if (limit_cycles < 0) return SHISO_ERR_SHAPE;
    if (limit_cycles > 10000000ll) limit_cycles = 10000000ll;
    bounded_wait_kernel<<<1, 32, 0, stream>>>((unsigned long long)limit_cycles, shiso_tc_status_word());
    return launch_status();
}
