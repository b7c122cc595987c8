// Test-only kernel: makes a bounded wait of the library's pipeline code run out, in the one form that is safe on a
// shared GPU -- a wait that gives up by itself and returns a status.  Nothing here faults, traps or spins for ever.
//
// One CTA initialises an mbarrier that nobody ever arrives on.  Two of its threads play two pipeline roles and call the
// very wait the GEMM kernels use (ptx::mbar_wait from csrc/ptx_sm100.cuh), compiled here with a 1 ms limit instead of
// the library's 2 s.  The first wait to time out raises the shared abort flag; the other role sees the flag (or times
// out itself) and leaves too.  The CTA then does what every GEMM kernel does at its end: it raises the per-device
// error flag, which odl_device_status turns into ODL_ERR_KERNEL_TIMEOUT and which makes later GEMM launches exit at
// once until it is cleared.  No copy is in flight, no TMEM is held, so there is nothing to clean up.
#define ODL_WAIT_NS 1000000ull  // 1 ms
#include <cuda_runtime.h>

#include "../../origindl_b200/csrc/ptx_sm100.cuh"

namespace
{
__global__ void wait_that_gives_up_kernel(int *device_err_flag, long long *report)
{
    __shared__ uint64_t never_completed;
    __shared__ int abort_flag;
    __shared__ int gave_up[2];
    if (threadIdx.x == 0)
    {
        abort_flag = 0;
        gave_up[0] = gave_up[1] = 0;
        odl::ptx::mbar_init(&never_completed, 1);
        odl::ptx::fence_mbar_init();
    }
    __syncthreads();
    const unsigned long long t0 = odl::ptx::globaltimer_ns();
    if (threadIdx.x == 0 || threadIdx.x == 32)  // two roles in two warps, like producer and MMA issuer
    {
        const bool completed = odl::ptx::mbar_wait(&never_completed, 0, &abort_flag);
        gave_up[threadIdx.x >> 5] = completed ? 0 : 1;
    }
    __syncthreads();
    if (threadIdx.x == 0)
    {
        report[0] = gave_up[0];
        report[1] = gave_up[1];
        report[2] = abort_flag;
        report[3] = static_cast<long long>(odl::ptx::globaltimer_ns() - t0);
        if (abort_flag && device_err_flag != nullptr)
            atomicExch(device_err_flag, 1);
    }
}
}  // namespace

// report: 4 x int64 on the device: role 0 gave up, role 1 gave up, abort flag, nanoseconds spent waiting.
extern "C" int odl_test_wait_that_gives_up(int *device_err_flag, long long *report, void *stream)
{
    wait_that_gives_up_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(device_err_flag, report);
    return static_cast<int>(cudaGetLastError());
}
