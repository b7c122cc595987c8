// functional::LinearOp on the fused kernels -- replaces src/operators/custom/linear.cpp of OriginDL.
//
// Forward  y = flatten(x) . W^T + b  (W [out, in], b [out]) is ONE launch (GEMM with the bias in its epilogue) instead of
// transpose + matmul + broadcast_to + add.  Backward -- which the reference leaves as "not implemented"
// (src/operators/custom/linear.cpp:116-121) -- is  gx = gy . W,  gW = gy^T . x,  gb = column sums of gy,  i.e. the chain
// Add::backward -> BroadcastTo::backward -> MatMul::backward of the unfused graph, computed without the two
// materialised transposes and with one pass over gy for the bias gradient.
// Tensors that are not contiguous float32 on a CUDA device take the same route through the Mat interface the reference
// uses, so the operator keeps working on the CPU backend and for the other dtypes.
#include "origin/operators/custom/linear.h"

#include "b200_glue.h"
#include "origin/core/operator.h"
#include "origin/core/tensor.h"
#include "origin/mat/origin/origin_mat.h"

namespace origin
{
namespace functional
{

namespace
{
bool fused_ok(const Mat &m)
{
    return m.device().type() == DeviceType::kCUDA && m.dtype() == DataType::kFloat32 && m.is_contiguous();
}
const float *fptr(const Mat &m)
{
    return static_cast<const OriginMat &>(m).data_ptr<float>();
}
float *fptr(Mat &m)
{
    return static_cast<OriginMat &>(m).data_ptr<float>();
}
size_t flat_features(const Shape &s)
{
    size_t f = 1;
    for (size_t i = 1; i < s.size(); ++i)
        f *= s[i];
    return f;
}
}  // namespace

std::vector<Tensor> LinearOp::forward(const std::vector<Tensor> &xs)
{
    const size_t expected = use_bias_ ? 3 : 2;
    if (unlikely(xs.size() != expected))
    {
        THROW_RUNTIME_ERROR("Linear operator requires {} inputs (x, weight{}), but got {}", expected, use_bias_ ? ", bias" : "",
                            xs.size());
    }
    const Tensor &x = xs[0], &weight = xs[1];
    const Shape xs_shape = x.shape(), ws = weight.shape();
    if (unlikely(xs_shape.size() < 2))
    {
        THROW_RUNTIME_ERROR("Linear forward: x must be 2D after flattening, but got shape {}", xs_shape.to_string());
    }
    if (unlikely(ws.size() != 2))
    {
        THROW_RUNTIME_ERROR("Linear forward: weight must be 2D (out_features, in_features), but got shape {}", ws.to_string());
    }
    const size_t M = xs_shape[0], K = flat_features(xs_shape), N = ws[0];
    if (unlikely(K != ws[1]))
    {
        THROW_RUNTIME_ERROR("Linear forward: feature mismatch - x has {} features, but weight expects {} features", K, ws[1]);
    }
    if (unlikely(N != static_cast<size_t>(out_features_)))
    {
        THROW_RUNTIME_ERROR("Linear forward: output feature mismatch - weight has {} out_features, but expected {}", N,
                            out_features_);
    }
    const Mat &xm = mat(x), &wm = mat(weight);
    const Mat *bm = use_bias_ ? &mat(xs[2]) : nullptr;
    if (fused_ok(xm) && fused_ok(wm) && (!bm || (fused_ok(*bm) && bm->elements() == N)))
    {
        b200::odl_ready(xm.device());
        auto y = std::make_unique<OriginMat>(Shape{M, N}, xm.dtype(), xm.device());
        b200::odl_check(odl_linear_forward(fptr(xm), nullptr, fptr(wm), nullptr, bm ? fptr(*bm) : nullptr, y->data_ptr<float>(),
                                           nullptr, (int64_t)M, (int64_t)N, (int64_t)K, ODL_W_OUT_IN, 0, b200::precision_mode(),
                                           nullptr),
                        "linear forward");
        return std::vector<Tensor>{convert_mat_to_tensor(std::move(y))};
    }
    // any other device / dtype: the unfused route through the Mat interface
    std::unique_ptr<Mat> x_flat = xs_shape.size() > 2 ? xm.reshape(Shape{M, K}) : nullptr;
    const Mat &x2               = x_flat ? *x_flat : xm;
    auto w_t                    = wm.transpose();
    auto y                      = x2.matmul(*w_t);
    if (bm)
    {
        auto b_full = bm->broadcast_to(y->shape());
        y           = *y + *b_full;
    }
    return std::vector<Tensor>{convert_mat_to_tensor(std::move(y))};
}

std::vector<Tensor> LinearOp::backward(const std::vector<Tensor> &gys)
{
    if (unlikely(gys.size() != 1))
    {
        THROW_RUNTIME_ERROR("Linear backward requires exactly 1 gradient, but got {}", gys.size());
    }
    const Tensor &x = this->inputs_[0], &weight = this->inputs_[1];
    const Shape xs_shape = x.shape(), ws = weight.shape();
    const size_t M = xs_shape[0], K = flat_features(xs_shape), N = ws[0];
    const Mat &xm = mat(x), &wm = mat(weight), &gm = mat(gys[0]);
    const Mat *bm = use_bias_ ? &mat(this->inputs_[2]) : nullptr;
    if (unlikely(gm.shape() != Shape({M, N})))
    {
        THROW_RUNTIME_ERROR("Linear backward: gradient has shape {}, expected ({}, {})", gm.shape().to_string(), M, N);
    }
    std::vector<Tensor> grads;
    if (fused_ok(xm) && fused_ok(wm) && fused_ok(gm) && (!bm || fused_ok(*bm)))
    {
        b200::odl_ready(xm.device());
        auto gx = std::make_unique<OriginMat>(xs_shape, xm.dtype(), xm.device());
        auto gw = std::make_unique<OriginMat>(ws, wm.dtype(), wm.device());
        std::unique_ptr<OriginMat> gb;
        if (bm)
            gb = std::make_unique<OriginMat>(bm->shape(), bm->dtype(), bm->device());
        b200::odl_check(odl_linear_backward(fptr(xm), nullptr, fptr(wm), nullptr, fptr(gm), nullptr, gx->data_ptr<float>(),
                                            gw->data_ptr<float>(), gb ? gb->data_ptr<float>() : nullptr, (int64_t)M, (int64_t)N,
                                            (int64_t)K, ODL_W_OUT_IN, b200::precision_mode(), nullptr),
                        "linear backward");
        grads.push_back(convert_mat_to_tensor(std::move(gx)));
        grads.push_back(convert_mat_to_tensor(std::move(gw)));
        if (gb)
            grads.push_back(convert_mat_to_tensor(std::move(gb)));
        return grads;
    }
    std::unique_ptr<Mat> x_flat = xs_shape.size() > 2 ? xm.reshape(Shape{M, K}) : nullptr;
    const Mat &x2               = x_flat ? *x_flat : xm;
    auto gx                     = gm.matmul(wm);  // [M, N] . [N, K]
    if (xs_shape.size() > 2)
        gx = gx->reshape(xs_shape);
    auto g_t = gm.transpose();
    auto gw  = g_t->matmul(x2);  // [N, M] . [M, K]
    grads.push_back(convert_mat_to_tensor(std::move(gx)));
    grads.push_back(convert_mat_to_tensor(std::move(gw)));
    if (bm)
    {
        auto gb = gm.sum_to(Shape{1, N});
        grads.push_back(convert_mat_to_tensor(gb->reshape(bm->shape())));
    }
    return grads;
}

Tensor custom_linear(const Tensor &x, const Tensor &weight, const Tensor &bias, int in_features, int out_features, bool use_bias)
{
    auto op = std::make_shared<LinearOp>(in_features, out_features, use_bias);
    return use_bias ? (*op)({x, weight, bias})[0] : (*op)({x, weight})[0];
}

Tensor custom_linear(const Tensor &x, const Tensor &weight, int in_features, int out_features)
{
    return custom_linear(x, weight, Tensor(), in_features, out_features, false);
}

}  // namespace functional
}  // namespace origin
