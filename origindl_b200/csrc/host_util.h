// Host-side helpers shared by the translation units of the library: last-error text and CUDA call checking.
#pragma once
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>

namespace odl
{

void set_last_error(const char *fmt, ...);
const char *get_last_error();

// Number of kernels this library has launched in the process (the benchmark reports the delta over its timed region).
extern long long g_launch_count;

// Per-device int the kernels raise when a bounded wait runs out.  Allocated by odl_init.
int *device_error_flag();

}  // namespace odl

#define ODL_CUDA_TRY(expr)                                                                                  \
    do                                                                                                      \
    {                                                                                                       \
        cudaError_t _e = (expr);                                                                            \
        if (_e != cudaSuccess)                                                                              \
        {                                                                                                   \
            ::odl::set_last_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
            return ::odl::kCudaError;                                                                       \
        }                                                                                                   \
    } while (0)
