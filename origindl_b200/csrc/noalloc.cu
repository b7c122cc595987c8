// Softmax-cross-entropy for callers that must not allocate device memory.
//
// The regular entry point (odl_softmax_cross_entropy) keeps one float per batch row between its two kernels and takes
// that scratch from the library's arena, which grows with cudaMalloc the first time a size is seen.  Some hosts cannot
// afford that: an application that handed the whole GPU to its own memory pool at start-up has nothing left for
// cudaMalloc to give, and a latency-critical loop cannot accept the device-wide synchronisation an allocation
// implies.  For them this file keeps the per-row scratch in a fixed array that is part of the library image.
//
// Cost and limits: every GPU that loads the library holds the array (256 KiB) until the process exits; at most
// ODL_STATIC_SOFTMAX_MAX_ROWS rows per call; all calls share the one array, so two calls that overlap on the GPU
// (different streams, or different host threads) race on it -- issue them on one stream.  Nothing in the array has to
// start at zero: each call overwrites rows [0, B) in its first kernel before its second kernel reads them, and never
// reads what an earlier call left behind.
#include <cuda_runtime.h>

#include <mutex>

#include "../../include/odl_b200.h"
#include "gemm_tc.cuh"
#include "host_util.h"
#include "internal.h"

namespace
{
// One float per batch row.  In host code this name is only a handle for cudaGetSymbolAddress, never a device
// address; kernels get the address resolved below.
static __device__ __align__(256) float g_static_row_loss[ODL_STATIC_SOFTMAX_MAX_ROWS];

constexpr int kMaxDevices            = 64;
float *g_scratch_addr[kMaxDevices]   = {};
std::mutex g_scratch_mu;

// Resolve the array's device address once per device, with that device current.
int static_scratch(float **out)
{
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    {
        odl::set_last_error("softmax_cross_entropy_static: cudaGetDevice failed or device index out of range: %s",
                            cudaGetErrorString(e));
        return odl::kCudaError;
    }
    std::lock_guard<std::mutex> lk(g_scratch_mu);
    if (!g_scratch_addr[dev])
    {
        void *p = nullptr;
        e       = cudaGetSymbolAddress(&p, g_static_row_loss);
        if (e != cudaSuccess || !p)
        {
            odl::set_last_error("softmax_cross_entropy_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            return odl::kCudaError;
        }
        g_scratch_addr[dev] = static_cast<float *>(p);
    }
    *out = g_scratch_addr[dev];
    return odl::kOk;
}
}  // namespace

extern "C" int odl_softmax_cross_entropy_static(const float *logits, const void *labels, int labels_are_int64, int64_t B,
                                                int64_t C, float *loss, float *dlogits, float grad_scale, void *stream)
{
    if (!odl::is_ready())
    {
        odl::set_last_error("odl_init has not been called");
        return odl::kNotInitialized;
    }
    if (B > ODL_STATIC_SOFTMAX_MAX_ROWS)
    {
        odl::set_last_error("softmax_cross_entropy_static: %lld rows exceed the fixed scratch of %d rows; use "
                            "odl_softmax_cross_entropy or split the batch",
                            (long long)B, ODL_STATIC_SOFTMAX_MAX_ROWS);
        return odl::kTooLarge;
    }
    float *scratch = nullptr;
    int rc         = static_scratch(&scratch);  // first call on a device: resolves the symbol, which also makes the
                                                // lazily loaded module image (and with it the array) resident
    if (rc)
        return rc;
    return odl::softmax_ce_launch(logits, labels_are_int64 ? nullptr : static_cast<const int32_t *>(labels),
                                  labels_are_int64 ? static_cast<const int64_t *>(labels) : nullptr, B, C, loss, dlogits,
                                  scratch, grad_scale, static_cast<cudaStream_t>(stream));
}
