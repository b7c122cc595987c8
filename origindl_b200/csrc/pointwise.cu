// Small element-wise kernels the operator layer needs around the hot path: same-shape add / subtract / multiply,
// scaling, y += alpha * x (gradient accumulation and the WeightDecay hook), fill, and a full reduction to a scalar.
// All are grid-stride loops over a grid of a multiple of the SM count; every arithmetic operation is rounded to fp32
// on its own (no fused multiply-add) so that results match the reference's chain of separate tensor operations.
#include <cuda_runtime.h>

#include "../../include/odl_b200.h"
#include "gemm_tc.cuh"
#include "host_util.h"
#include "internal.h"

namespace odl
{
namespace
{
constexpr int kBlock = 256;
inline int grid_of(int64_t n)
{
    int64_t b = (n + kBlock - 1) / kBlock;
    if (b > 148 * 8)
        b = 148 * 8;
    return b < 1 ? 1 : static_cast<int>(b);
}

__global__ void binary_kernel(int op, const float *__restrict__ x, const float *__restrict__ y, float *__restrict__ out,
                              int64_t n)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    {
        const float a = x[i], b = y[i];
        out[i] = op == 0 ? __fadd_rn(a, b) : (op == 1 ? __fsub_rn(a, b) : __fmul_rn(a, b));
    }
}

__global__ void scale_kernel(const float *__restrict__ x, float alpha, float *__restrict__ out, int64_t n)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
        out[i] = __fmul_rn(x[i], alpha);
}

__global__ void axpy_kernel(float alpha, const float *__restrict__ x, float *__restrict__ y, int64_t n)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
        y[i] = __fadd_rn(y[i], __fmul_rn(x[i], alpha));
}

__global__ void fill_kernel(float *__restrict__ out, float v, int64_t n)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
        out[i] = v;
}

// One block, fixed summation order (deterministic): per-thread strided partial sums, then a shared-memory tree.
__global__ void __launch_bounds__(1024) sum_all_kernel(const float *__restrict__ x, float *__restrict__ out, int64_t n)
{
    __shared__ float red[1024];
    float s = 0.f;
    for (int64_t i = threadIdx.x; i < n; i += 1024)
        s += x[i];
    red[threadIdx.x] = s;
    __syncthreads();
    for (int o = 512; o > 0; o >>= 1)
    {
        if (threadIdx.x < o)
            red[threadIdx.x] += red[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0)
        out[0] = red[0];
}

int check_launch(const char *name)
{
    ++g_launch_count;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
    {
        set_last_error("%s launch failed: %s", name, cudaGetErrorString(e));
        return kCudaError;
    }
    return kOk;
}
}  // namespace
}  // namespace odl

using namespace odl;
#define ST(x) static_cast<cudaStream_t>(x)

extern "C" {

int odl_binary(int op, const float *x, const float *y, float *out, int64_t n, void *stream)
{
    if (op < 0 || op > 2 || !x || !y || !out || n <= 0)
    {
        set_last_error("binary: invalid argument (op=%d n=%lld)", op, (long long)n);
        return kInvalidArgument;
    }
    binary_kernel<<<grid_of(n), kBlock, 0, ST(stream)>>>(op, x, y, out, n);
    return check_launch("binary_kernel");
}

int odl_scale(const float *x, float alpha, float *out, int64_t n, void *stream)
{
    if (!x || !out || n <= 0)
    {
        set_last_error("scale: invalid argument");
        return kInvalidArgument;
    }
    scale_kernel<<<grid_of(n), kBlock, 0, ST(stream)>>>(x, alpha, out, n);
    return check_launch("scale_kernel");
}

int odl_axpy(float alpha, const float *x, float *y, int64_t n, void *stream)
{
    if (!x || !y || n <= 0)
    {
        set_last_error("axpy: invalid argument");
        return kInvalidArgument;
    }
    axpy_kernel<<<grid_of(n), kBlock, 0, ST(stream)>>>(alpha, x, y, n);
    return check_launch("axpy_kernel");
}

int odl_fill(float *out, float value, int64_t n, void *stream)
{
    if (!out || n <= 0)
    {
        set_last_error("fill: invalid argument");
        return kInvalidArgument;
    }
    fill_kernel<<<grid_of(n), kBlock, 0, ST(stream)>>>(out, value, n);
    return check_launch("fill_kernel");
}

int odl_sum_all(const float *x, float *out, int64_t n, void *stream)
{
    if (!x || !out || n <= 0)
    {
        set_last_error("sum_all: invalid argument");
        return kInvalidArgument;
    }
    sum_all_kernel<<<1, 1024, 0, ST(stream)>>>(x, out, n);
    return check_launch("sum_all_kernel");
}

}  // extern "C"
