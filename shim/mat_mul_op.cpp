// functional::MatMul on the B200 GEMM -- replaces src/operators/math/mat_mul.cpp of OriginDL.
//
// Forward goes through Mat::matmul as before (origin::cuda::matmul of this shim on a GPU).  Backward of the 2-D product
// y = x . w on contiguous float32 CUDA tensors is two GEMMs that read the operands where they lie:
//     gx = gy . w^T   (w read as an [N, K]-stored right operand)      gw = x^T . gy   (x read as a [K, M]-stored left operand)
// instead of the reference's two materialised transposes followed by two GEMMs (src/operators/math/mat_mul.cpp:171-177,
// src/mat/origin/cuda/shape/transpose.cu:191-221).  Every other case (CPU, other dtypes, batched) keeps that route.
#include "origin/operators/math/mat_mul.h"

#include "b200_glue.h"
#include "origin/core/operator.h"
#include "origin/core/tensor.h"
#include "origin/mat/origin/origin_mat.h"
#include "origin/mat/type_promotion.h"

namespace origin
{
namespace functional
{

namespace
{
// 0-d and 1-d operands act as matrices: a left vector is a row, a right vector is a column.
Tensor as_matrix(const Tensor &t, bool left)
{
    const Shape s = t.shape();
    if (s.size() == 0)
        return t.reshape(Shape{1, 1});
    if (s.size() == 1)
        return left ? t.reshape(Shape{1, s[0]}) : t.reshape(Shape{s[0], 1});
    return t;
}

bool fused_ok(const Mat &m)
{
    return m.device().type() == DeviceType::kCUDA && m.dtype() == DataType::kFloat32 && m.is_contiguous() &&
           m.shape().size() == 2;
}
}  // namespace

std::vector<Tensor> MatMul::forward(const std::vector<Tensor> &xs)
{
    if (unlikely(xs.size() != 2))
    {
        THROW_RUNTIME_ERROR("MatMul operator requires exactly 2 inputs, but got {}", xs.size());
    }
    if (unlikely(xs[0].shape().elements() == 0 || xs[1].shape().elements() == 0))
    {
        THROW_RUNTIME_ERROR("MatMul forward: input shapes invalid - xs[0].shape() = {}, xs[1].shape() = {}",
                            xs[0].shape().to_string(), xs[1].shape().to_string());
    }
    Tensor a = as_matrix(xs[0], true), b = as_matrix(xs[1], false);
    const Shape sa = a.shape(), sb = b.shape();
    // supported: 2-D x 2-D, 3-D x 2-D, 3-D x 3-D (same batch); the reduced extents must agree
    const bool ranks_ok = (sa.size() == 2 && sb.size() == 2) || (sa.size() == 3 && (sb.size() == 2 || sb.size() == 3));
    if (unlikely(!ranks_ok))
    {
        THROW_RUNTIME_ERROR("MatMul forward: unsupported shape combination - x0.shape() = {}, x1.shape() = {}", sa.to_string(),
                            sb.to_string());
    }
    if (unlikely(sa.size() == 3 && sb.size() == 3 && sa[0] != sb[0]))
    {
        THROW_RUNTIME_ERROR("MatMul forward: batch size mismatch - x0.shape() = {}, x1.shape() = {}", sa.to_string(),
                            sb.to_string());
    }
    if (unlikely(sa[sa.size() - 1] != sb[sb.size() - 2]))
    {
        THROW_RUNTIME_ERROR("MatMul forward: dimension mismatch - x0.shape() = {}, x1.shape() = {}", sa.to_string(),
                            sb.to_string());
    }
    auto [a_p, b_p] = TypePromotion::promote_tensors_maybe_owned(a, b);
    a               = Tensor(a_p);
    b               = Tensor(b_p);
    return std::vector<Tensor>{convert_mat_to_tensor(mat(a).matmul(mat(b)))};
}

std::vector<Tensor> MatMul::backward(const std::vector<Tensor> &gys)
{
    if (unlikely(gys.size() != 1))
    {
        THROW_RUNTIME_ERROR("MatMul backward requires exactly 1 gradient, but got {}", gys.size());
    }
    auto [x_p, w_p] = TypePromotion::promote_tensors_maybe_owned(this->inputs_[0], this->inputs_[1]);
    Tensor x = as_matrix(Tensor(x_p), true), w = as_matrix(Tensor(w_p), false), gy = gys[0];
    if (unlikely(x.shape().size() < 2 || w.shape().size() < 2))
    {
        THROW_RUNTIME_ERROR("MatMul backward: after reshape, shapes must be at least 2D - x.shape() = {}, w.shape() = {}",
                            x.shape().to_string(), w.shape().to_string());
    }
    const Mat &xm = mat(x), &wm = mat(w), &gm = mat(gy);
    if (fused_ok(xm) && fused_ok(wm) && fused_ok(gm) && gm.shape() == Shape({xm.shape()[0], wm.shape()[1]}))
    {
        const int64_t M = (int64_t)xm.shape()[0], K = (int64_t)xm.shape()[1], N = (int64_t)wm.shape()[1];
        b200::odl_ready(xm.device());
        auto gx        = std::make_unique<OriginMat>(xm.shape(), xm.dtype(), xm.device());
        auto gw        = std::make_unique<OriginMat>(wm.shape(), wm.dtype(), wm.device());
        const float *X = static_cast<const OriginMat &>(xm).data_ptr<float>();
        const float *W = static_cast<const OriginMat &>(wm).data_ptr<float>();
        const float *G = static_cast<const OriginMat &>(gm).data_ptr<float>();
        const int prec = b200::precision_mode();
        // gx[M,K] = gy[M,N] . w^T : w is stored [K,N] = "[out, reduce]" for this product -> transB
        b200::odl_check(odl_gemm_ex(0, 1, M, K, N, G, nullptr, N, W, nullptr, N, gx->data_ptr<float>(), nullptr, K, nullptr,
                                    nullptr, 0, nullptr, 0, prec, nullptr),
                        "matmul backward (gx)");
        // gw[K,N] = x^T . gy : x is stored [M,K] = "[reduce, out]" for this product -> transA
        b200::odl_check(odl_gemm_ex(1, 0, K, N, M, X, nullptr, K, G, nullptr, N, gw->data_ptr<float>(), nullptr, N, nullptr,
                                    nullptr, 0, nullptr, 0, prec, nullptr),
                        "matmul backward (gw)");
        return std::vector<Tensor>{convert_mat_to_tensor(std::move(gx)), convert_mat_to_tensor(std::move(gw))};
    }
    auto w_t = wm.transpose();
    auto x_t = xm.transpose();
    auto gx  = gm.matmul(*w_t);
    auto gw  = x_t->matmul(gm);
    return std::vector<Tensor>{convert_mat_to_tensor(std::move(gx)), convert_mat_to_tensor(std::move(gw))};
}

Tensor matmul(const std::vector<Tensor> &xs)
{
    auto op = std::make_shared<MatMul>();
    return (*op)(xs)[0];
}

Tensor matmul(const Tensor &lhs, const Tensor &rhs)
{
    return matmul({lhs, rhs});
}

Tensor mat_mul(const Tensor &lhs, const Tensor &rhs)
{
    return matmul(lhs, rhs);
}

}  // namespace functional
}  // namespace origin
