// Self-test of the bounded-wait / status-word path that every kernel of the library relies on.
//
// One small CTA initialises an mbarrier that nobody ever arrives on, waits for it with the same
// bounded wait the fused GEMM uses (ptx.cuh: mbar_wait) but with a caller-chosen limit, and when
// the limit runs out records STATUS_SELFTEST_WAIT in the device status word and returns. The
// kernel always ends by itself; the context stays usable; nf4b200_device_status then reports
// NF4B200_EDEVICE. Nothing here faults, traps or spins without a limit.
#include <cuda_runtime.h>

#include "kernels.h"
#include "ptx.cuh"

namespace nf4 {

__global__ void __launch_bounds__(32)
selftest_wait_kernel(int* status, unsigned long long limit_ns) {
    __shared__ __align__(8) unsigned long long bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_flag = 0;
        fence_barrier_init();
    }
    __syncthreads();
    // phase 0 of a barrier with one expected arrival that never comes
    const bool done = mbar_wait(smem_u32(&bar), 0u, &abort_flag, limit_ns);
    if (!done && threadIdx.x == 0) atomicCAS(status, 0, STATUS_SELFTEST_WAIT);
}

cudaError_t launch_selftest_wait(unsigned long long limit_ns, cudaStream_t stream) {
    int* status = device_status_word();
    if (status == nullptr) return cudaErrorInvalidDevice;
    selftest_wait_kernel<<<1, 32, 0, stream>>>(status, limit_ns);
    return cudaGetLastError();
}

}  // namespace nf4
