// A kernel whose only wait is never satisfied, for the test of the bounded-wait path.
//
// Every mbarrier wait of the tensor-core kernels goes through mbar_wait (tma_helpers.cuh), which gives up after
// RS_WAIT_LIMIT_NS, sets RS_STATUS_WAIT_EXPIRED and lets the kernel return, so that a logic error cannot hang the
// device.  In a correct run that path never executes.  This file builds into a library of its own, compiled with
// a limit of 2 ms, which the engine never loads: one CTA initialises a barrier that expects one arrival, nobody
// arrives, the wait runs out after 2 ms, the status bit is set and the kernel ends normally.  Nothing faults and
// nothing hangs; the context stays usable, which is what the test then checks with an ordinary step.
#include "tma_helpers.cuh"

namespace {
__global__ void wait_probe_kernel(int* status, int* outcome) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned long long t0 = global_ns();
        const bool ok = mbar_wait(smem_u32(&bar), 0, &abort_flag, status);      // phase 0 never completes
        outcome[0] = ok ? 1 : 0;
        outcome[1] = (int)((global_ns() - t0) / 1000ull);                       // microseconds waited
    }
    __syncthreads();
}
}  // namespace

RS_EXPORT unsigned long long rs_wait_probe_limit_ns() { return RS_WAIT_LIMIT_NS; }

// outcome[0] = 1 if the wait was satisfied (it cannot be), 0 if it gave up; outcome[1] = microseconds it waited.
RS_EXPORT int rs_wait_probe(int* status, int* outcome, void* stream) {
    wait_probe_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(status, outcome);
    return rs_launch_result();
}
