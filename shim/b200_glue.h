// Glue shared by the shim's translation units: lazy odl_init, status -> exception, run-time switches.
#pragma once
#include <cstdlib>
#include <mutex>
#include <string>

#include "odl_b200.h"
#include "origin/mat/basic_types.h"
#include "origin/utils/branch_prediction.h"
#include "origin/utils/exception.h"

namespace origin
{
namespace b200
{

// Binds the library to the tensor's GPU on first use (one device per process, like odl_init itself).
inline void odl_ready(const Device &device)
{
    static std::once_flag once;
    static int status = ODL_OK;
    std::call_once(once, [&] { status = odl_init(device.index()); });
    if (unlikely(status != ODL_OK))
    {
        THROW_RUNTIME_ERROR("B200 backend: odl_init failed: {}", odl_last_error());
    }
}

// ODL_ERR_INVALID_ARGUMENT -> std::invalid_argument, anything else non-zero -> std::runtime_error, both with the
// reference's "[file:func:line]" prefix (include/origin/utils/exception.h:37-60).
inline void odl_check(int status, const char *what)
{
    if (likely(status == ODL_OK))
        return;
    if (status == ODL_ERR_INVALID_ARGUMENT)
    {
        THROW_INVALID_ARG("{}: {}", what, odl_last_error());
    }
    THROW_RUNTIME_ERROR("{} failed (odl status {}): {}", what, status, odl_last_error());
}

// ORIGIN_MATMUL_PRECISION = 3xtf32 (default: fp32-class accuracy, three tf32 MMAs per product) | tf32.
// Read once, next to the reference's own ORIGIN_KERNEL_ALGO (include/origin/utils/env_config.h:16-21).
inline int precision_mode()
{
    static const int mode = [] {
        const char *v = std::getenv("ORIGIN_MATMUL_PRECISION");
        return (v && std::string(v) == "tf32") ? ODL_PRECISION_TF32 : ODL_PRECISION_3XTF32;
    }();
    return mode;
}

// ORIGIN_CONV2D_GRADIENT = reference (default: conv2d_backward reinterprets the NCHW gradient buffer as [N*OH*OW, OC]
// rows, which is what the reference computes, src/mat/origin/cuda/conv/conv2d.cu:714) | true (the gradient of the
// forward pass: the buffer is permuted instead).  The two agree when OC == 1, OH*OW == 1 or gy is constant.
inline int conv_gradient_layout()
{
    static const int layout = [] {
        const char *v = std::getenv("ORIGIN_CONV2D_GRADIENT");
        return (v && std::string(v) == "true") ? 0 : 1;
    }();
    return layout;
}

}  // namespace b200
}  // namespace origin
