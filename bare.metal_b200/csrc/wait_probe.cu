// Self-test of the bounded wait every tensor-core kernel of this backend relies on (mbar_wait in ptx_sm100.cuh): one CTA waits on an
// mbarrier that nothing ever arrives at. This translation unit compiles the wait with a 2 ms limit instead of the kernels' 1 s, so
// the wait runs out at once: the waiter raises the CTA's abort flag, the kernel stores a status code in the context's error word and
// returns normally. Nothing faults, traps or hangs; the context stays usable, which the caller checks by running real work next.
#define BMB_WAIT_LIMIT_NS 2000000ull
#include "ptx_sm100.cuh"

namespace bmb {

constexpr int WAIT_PROBE_CODE = 1999;   // same range as the GEMM's 1000 + CTA index codes

__global__ void wait_probe_kernel(int* err) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) (void)mbar_wait(&bar, 0, &abort_flag);   // phase 0 never completes: no thread arrives
    __syncthreads();
    if (threadIdx.x == 0 && abort_flag && err) atomicExch(err, WAIT_PROBE_CODE);
}

int wait_probe_launch(int* err, cudaStream_t st) {
    wait_probe_kernel<<<1, 64, 0, st>>>(err);
    return cudaPeekAtLastError() == cudaSuccess ? 0 : -7;
}

}  // namespace bmb
