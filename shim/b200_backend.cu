// origin::cuda:: free functions of the dense hot path, implemented on libodl_b200.so.
//
// A maintainer of OriginDL builds liboriginmat_cuda / liborigindl with THIS file in place of
//     src/mat/origin/cuda/math/mat_mul.cu     (matmul)
//     src/mat/origin/cuda/conv/conv2d.cu      (im2col, col2im, conv2d, conv2d_backward)
//     src/mat/origin/cuda/activation/relu.cu  (relu)
//     src/mat/origin/cuda/math/sum_to.cu      (sum_to)
// and links libodl_b200.so.  The signatures are the reference's own (include/origin/mat/origin/cuda/cuda_ops.cuh:186,
// :264, :312, :335-383), so OriginMat's device switch (src/mat/origin/origin_mat.cpp:659-679 and its siblings) links
// unchanged and every Operator above it runs on the B200 kernels.  Outputs are allocated as OriginMat(shape, dtype,
// device) exactly like the files replaced (Storage -> MemoryPool); validation failures throw what the reference throws
// (THROW_INVALID_ARG / THROW_RUNTIME_ERROR); a non-zero odl status becomes a runtime_error carrying odl_last_error().
//
// fp32 goes to the tcgen05 kernels.  The reference templates these entry points over six dtypes; the other five keep
// working through the small generic kernels at the end of this file (they are not on the hot path and make no speed
// claim).  Everything runs on the legacy default stream, like every launch of the reference.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdlib>
#include <functional>
#include <memory>
#include <mutex>
#include <vector>

#include "b200_glue.h"
#include "odl_b200.h"
#include "origin/mat/origin/cuda/cuda_ops.cuh"
#include "origin/mat/origin/cuda/cuda_utils.cuh"
#include "origin/mat/origin/device_common/type_dispatcher.h"
#include "origin/mat/origin/origin_mat.h"
#include "origin/mat/origin/origin_mat_utils.h"
#include "origin/utils/branch_prediction.h"
#include "origin/utils/conv_utils.h"
#include "origin/utils/exception.h"

namespace origin
{
namespace cuda
{

namespace
{
using b200::conv_gradient_layout;
using b200::odl_check;
using b200::odl_ready;
using b200::precision_mode;

const OriginMat &as_contiguous(const OriginMat &m, std::unique_ptr<Mat> &keep)
{
    if (likely(m.is_contiguous()))
        return m;
    keep = m.contiguous();
    return static_cast<const OriginMat &>(*keep);
}

constexpr int kBlock = 256;
inline unsigned blocks_for(size_t n)
{
    return static_cast<unsigned>((n + kBlock - 1) / kBlock);
}

// ---- generic kernels for the dtypes the tensor-core path does not take -----------------------------------------------
template <typename T>
__global__ void generic_matmul_kernel(const T *a, const T *b, T *c, int M, int N, int K)
{
    __shared__ T ta[16][16], tb[16][17];
    const int row = blockIdx.y * 16 + threadIdx.y, col = blockIdx.x * 16 + threadIdx.x;
    T acc = T(0);
    for (int k0 = 0; k0 < K; k0 += 16)
    {
        ta[threadIdx.y][threadIdx.x] = (row < M && k0 + threadIdx.x < K) ? a[static_cast<size_t>(row) * K + k0 + threadIdx.x] : T(0);
        tb[threadIdx.y][threadIdx.x] = (k0 + threadIdx.y < K && col < N) ? b[static_cast<size_t>(k0 + threadIdx.y) * N + col] : T(0);
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 16; ++k)
            acc += ta[threadIdx.y][k] * tb[k][threadIdx.x];
        __syncthreads();
    }
    if (row < M && col < N)
        c[static_cast<size_t>(row) * N + col] = acc;
}

template <typename T>
__global__ void generic_relu_kernel(const T *x, T *y, size_t n)
{
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n)
        y[i] = x[i] > T(0) ? x[i] : T(0);
}

struct ConvGeom
{
    int N, C, H, W, KH, KW, SH, SW, PH, PW, OH, OW;
};

// One thread per element of the column tensor; reads the image directly (zero outside it): no padded copy.
// to_matrix: col[(n*OH+oh)*OW+ow][(c*KH+kh)*KW+kw], else col[n][c][kh][kw][oh][ow].
template <typename T>
__global__ void generic_im2col_kernel(const T *img, T *col, ConvGeom g, bool to_matrix, size_t total)
{
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= total)
        return;
    size_t r = i;
    int n, c, kh, kw, oh, ow;
    if (to_matrix)
    {
        kw = r % g.KW, r /= g.KW, kh = r % g.KH, r /= g.KH, c = r % g.C, r /= g.C;
        ow = r % g.OW, r /= g.OW, oh = r % g.OH, n = static_cast<int>(r / g.OH);
    }
    else
    {
        ow = r % g.OW, r /= g.OW, oh = r % g.OH, r /= g.OH, kw = r % g.KW, r /= g.KW;
        kh = r % g.KH, r /= g.KH, c = r % g.C, n = static_cast<int>(r / g.C);
    }
    const int h = oh * g.SH - g.PH + kh, w = ow * g.SW - g.PW + kw;
    col[i] = (h >= 0 && h < g.H && w >= 0 && w < g.W) ? img[((static_cast<size_t>(n) * g.C + c) * g.H + h) * g.W + w] : T(0);
}

// One thread per image element gathers the column entries that map to it, kh then kw ascending (no atomics).
template <typename T>
__global__ void generic_col2im_kernel(const T *col, T *img, ConvGeom g, bool to_matrix, size_t total)
{
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= total)
        return;
    size_t r    = i;
    const int w = r % g.W;
    r /= g.W;
    const int h = r % g.H;
    r /= g.H;
    const int c = r % g.C, n = static_cast<int>(r / g.C);
    T acc = T(0);
    for (int kh = 0; kh < g.KH; ++kh)
    {
        const int th = h + g.PH - kh;
        if (th < 0 || th % g.SH)
            continue;
        const int oh = th / g.SH;
        if (oh >= g.OH)
            continue;
        for (int kw = 0; kw < g.KW; ++kw)
        {
            const int tw = w + g.PW - kw;
            if (tw < 0 || tw % g.SW)
                continue;
            const int ow = tw / g.SW;
            if (ow >= g.OW)
                continue;
            const size_t at = to_matrix
                                  ? ((static_cast<size_t>(n) * g.OH + oh) * g.OW + ow) * (static_cast<size_t>(g.C) * g.KH * g.KW) +
                                        (static_cast<size_t>(c) * g.KH + kh) * g.KW + kw
                                  : ((((static_cast<size_t>(n) * g.C + c) * g.KH + kh) * g.KW + kw) * g.OH + oh) * g.OW + ow;
            acc += col[at];
        }
    }
    img[i] = acc;
}

ConvGeom conv_geom(const Shape &img, std::pair<int, int> k, std::pair<int, int> s, std::pair<int, int> p, const char *who)
{
    if (unlikely(img.size() != 4))
    {
        THROW_INVALID_ARG("{}: image must be 4D (N, C, H, W), but got shape {}", who, img.to_string());
    }
    ConvGeom g{(int)img[0], (int)img[1], (int)img[2], (int)img[3], k.first, k.second, s.first, s.second, p.first, p.second, 0, 0};
    g.OH = get_conv_outsize(g.H, g.KH, g.SH, g.PH);
    g.OW = get_conv_outsize(g.W, g.KW, g.SW, g.PW);
    if (unlikely(g.OH <= 0 || g.OW <= 0))
    {
        THROW_INVALID_ARG("{}: invalid output size OH={}, OW={} for input H={}, W={}, kernel=({},{}), stride=({},{}), pad=({},{})",
                          who, g.OH, g.OW, g.H, g.W, g.KH, g.KW, g.SH, g.SW, g.PH, g.PW);
    }
    return g;
}

bool odl_conv_form(const ConvGeom &g, DataType dt)
{
    return dt == DataType::kFloat32 && g.SH == g.SW && g.PH == g.PW;
}
}  // namespace

// ---- matmul: include/origin/mat/origin/cuda/cuda_ops.cuh:264 ----------------------------------------------------------
std::unique_ptr<Mat> matmul(const OriginMat &a, const OriginMat &b)
{
    VALIDATE_SAME_DTYPE(a, b);
    VALIDATE_SAME_CUDA_DEVICE(a, b);
    std::unique_ptr<Mat> keep_a, keep_b;
    const OriginMat &A = as_contiguous(a, keep_a);
    const OriginMat &B = as_contiguous(b, keep_b);
    const Shape sa = A.shape(), sb = B.shape();
    if (unlikely(sa.size() < 2 || sb.size() < 2))
    {
        THROW_INVALID_ARG("MatMul requires at least 2D tensors, got shapes {} and {}", sa.to_string(), sb.to_string());
    }
    const size_t M = sa[sa.size() - 2], K = sa[sa.size() - 1], K2 = sb[sb.size() - 2], N = sb[sb.size() - 1];
    if (unlikely(K != K2))
    {
        THROW_INVALID_ARG("MatMul dimension mismatch: {} vs {}", sa.to_string(), sb.to_string());
    }
    size_t batch      = 1;
    bool b_batched    = false;
    Shape out_shape{M, N};
    if (sa.size() == 3 && (sb.size() == 2 || sb.size() == 3))
    {
        batch     = sa[0];
        b_batched = sb.size() == 3;
        out_shape = Shape{batch, M, N};
    }
    else if (unlikely(!(sa.size() == 2 && sb.size() == 2)))
    {
        THROW_RUNTIME_ERROR("Complex broadcasting not yet implemented for CUDA matmul");
    }
    auto result = std::make_unique<OriginMat>(out_shape, A.dtype(), A.device());
    if (likely(A.dtype() == DataType::kFloat32))
    {
        odl_ready(A.device());
        odl_check(odl_matmul(A.data_ptr<float>(), B.data_ptr<float>(), result->data_ptr<float>(), (int64_t)M, (int64_t)N,
                             (int64_t)K, (int64_t)batch, b_batched ? 1 : 0, precision_mode(), nullptr),
                  "matmul");
        return result;
    }
    device_common::TypeDispatcher::dispatch_void(A.dtype(), [&]<typename T>() {
        const dim3 block(16, 16), grid((unsigned)((N + 15) / 16), (unsigned)((M + 15) / 16));
        for (size_t i = 0; i < batch; ++i)
            generic_matmul_kernel<T><<<grid, block>>>(A.data_ptr<T>() + i * M * K, B.data_ptr<T>() + (b_batched ? i * K * N : 0),
                                                      result->data_ptr<T>() + i * M * N, (int)M, (int)N, (int)K);
    });
    CUDA_CHECK_ASYNC();
    return result;
}

// ---- relu: cuda_ops.cuh:186 -----------------------------------------------------------------------------------------
std::unique_ptr<Mat> relu(const OriginMat &mat, OriginMat *out)
{
    VALIDATE_CUDA_DEVICE(mat);
    std::unique_ptr<OriginMat> fresh;
    OriginMat *dst = out;
    if (out != nullptr)
    {
        if (unlikely(out->shape() != mat.shape() || out->dtype() != mat.dtype() || out->device() != mat.device()))
        {
            THROW_INVALID_ARG("Output tensor mismatch. Expected shape={}, dtype={}, device={}, but got shape={}, dtype={}, device={}",
                              mat.shape().to_string(), dtype_to_string(mat.dtype()), mat.device().to_string(),
                              out->shape().to_string(), dtype_to_string(out->dtype()), out->device().to_string());
        }
    }
    else
    {
        fresh = std::make_unique<OriginMat>(mat.shape(), mat.dtype(), mat.device());
        dst   = fresh.get();
    }
    const size_t n = mat.elements();
    if (n == 0)
        return fresh;
    if (likely(mat.dtype() == DataType::kFloat32))
    {
        odl_ready(mat.device());
        odl_check(odl_relu_forward(mat.data_ptr<float>(), dst->data_ptr<float>(), (int64_t)n, nullptr), "relu");
        return fresh;
    }
    device_common::TypeDispatcher::dispatch_void(mat.dtype(), [&]<typename T>() {
        generic_relu_kernel<T><<<blocks_for(n), kBlock>>>(mat.data_ptr<T>(), dst->data_ptr<T>(), n);
    });
    CUDA_CHECK_ASYNC();
    return fresh;
}

// ---- sum_to: cuda_ops.cuh:312.  {M, N} -> {1, N} (the bias gradient of BroadcastTo::backward) is one ordered column-sum
//      pass; it has no limit on N (the reference's axis sum launches one block of N threads and fails above 1024).
std::unique_ptr<Mat> sum_to(const OriginMat &mat, const Shape &target_shape)
{
    VALIDATE_CUDA_DEVICE(mat);
    const Shape in = mat.shape();
    if (in == target_shape)
        return std::make_unique<OriginMat>(mat);
    if (unlikely(target_shape.elements() > mat.elements()))
    {
        THROW_RUNTIME_ERROR("sum_to: Target shape {} cannot have more elements than source tensor {}", target_shape.elements(),
                            mat.elements());
    }
    const bool rows_to_one = in.size() == 2 && in[0] > 1 && mat.dtype() == DataType::kFloat32 && mat.is_contiguous() &&
                             target_shape.size() == 2 && target_shape[0] == 1 && target_shape[1] == in[1];
    if (rows_to_one)
    {
        odl_ready(mat.device());
        auto result = std::make_unique<OriginMat>(target_shape, mat.dtype(), mat.device());
        odl_check(odl_sum_to_row(mat.data_ptr<float>(), result->data_ptr<float>(), (int64_t)in[0], (int64_t)in[1], nullptr),
                  "sum_to");
        return result;
    }
    // every other form: sum the axes that collapse (target extent 1, or missing on the right), highest axis first so the
    // remaining axis numbers stay valid, then give the result the target's shape
    std::vector<int> axes;
    for (size_t i = 0; i < std::min(in.size(), target_shape.size()); ++i)
        if (target_shape[i] == 1 && in[i] > 1)
            axes.push_back(static_cast<int>(i));
    for (size_t i = target_shape.size(); i < in.size(); ++i)
        axes.push_back(static_cast<int>(i));
    std::sort(axes.begin(), axes.end(), std::greater<int>());
    std::unique_ptr<Mat> cur = std::make_unique<OriginMat>(mat);
    for (int ax : axes)
        cur = static_cast<const OriginMat &>(*cur).sum(ax);
    if (cur->shape() != target_shape)
        cur = cur->reshape(target_shape);
    return cur;
}

// ---- im2col / col2im: cuda_ops.cuh:335, :349 --------------------------------------------------------------------------
std::unique_ptr<Mat> im2col(const OriginMat &img, std::pair<int, int> kernel_size, std::pair<int, int> stride,
                            std::pair<int, int> pad, bool to_matrix)
{
    VALIDATE_CUDA_DEVICE(img);
    std::unique_ptr<Mat> keep;
    const OriginMat &x = as_contiguous(img, keep);
    const ConvGeom g   = conv_geom(x.shape(), kernel_size, stride, pad, "im2col");
    const size_t N = g.N, C = g.C, KH = g.KH, KW = g.KW, OH = g.OH, OW = g.OW;
    const Shape out_shape = to_matrix ? Shape{N * OH * OW, C * KH * KW} : Shape{N, C, KH, KW, OH, OW};
    auto result           = std::make_unique<OriginMat>(out_shape, x.dtype(), x.device());
    if (to_matrix && odl_conv_form(g, x.dtype()) && (C * KH * KW) % 4 == 0)
    {
        odl_ready(x.device());
        odl_check(odl_im2col(x.data_ptr<float>(), result->data_ptr<float>(), g.N, g.C, g.H, g.W, g.KH, g.KW, g.SH, g.PH, nullptr),
                  "im2col");
        return result;
    }
    const size_t total = result->elements();
    device_common::TypeDispatcher::dispatch_void(x.dtype(), [&]<typename T>() {
        generic_im2col_kernel<T><<<blocks_for(total), kBlock>>>(x.data_ptr<T>(), result->data_ptr<T>(), g, to_matrix, total);
    });
    CUDA_CHECK_ASYNC();
    return result;
}

std::unique_ptr<Mat> col2im(const OriginMat &col, const Shape &input_shape, std::pair<int, int> kernel_size,
                            std::pair<int, int> stride, std::pair<int, int> pad, bool to_matrix)
{
    VALIDATE_CUDA_DEVICE(col);
    std::unique_ptr<Mat> keep;
    const OriginMat &c = as_contiguous(col, keep);
    const ConvGeom g   = conv_geom(input_shape, kernel_size, stride, pad, "col2im");
    const size_t want  = static_cast<size_t>(g.N) * g.OH * g.OW * g.C * g.KH * g.KW;
    if (unlikely(c.elements() != want))
    {
        THROW_INVALID_ARG("col2im: column tensor {} does not match input shape {} with kernel=({},{}), stride=({},{}), pad=({},{})",
                          c.shape().to_string(), input_shape.to_string(), g.KH, g.KW, g.SH, g.SW, g.PH, g.PW);
    }
    auto result = std::make_unique<OriginMat>(input_shape, c.dtype(), c.device());
    if (to_matrix && odl_conv_form(g, c.dtype()))
    {
        odl_ready(c.device());
        odl_check(odl_col2im(c.data_ptr<float>(), result->data_ptr<float>(), g.N, g.C, g.H, g.W, g.KH, g.KW, g.SH, g.PH, nullptr),
                  "col2im");
        return result;
    }
    const size_t total = result->elements();
    device_common::TypeDispatcher::dispatch_void(c.dtype(), [&]<typename T>() {
        generic_col2im_kernel<T><<<blocks_for(total), kBlock>>>(c.data_ptr<T>(), result->data_ptr<T>(), g, to_matrix, total);
    });
    CUDA_CHECK_ASYNC();
    return result;
}

// ---- conv2d / conv2d_backward: cuda_ops.cuh:363, :376 -----------------------------------------------------------------
namespace
{
ConvGeom conv_checked(const OriginMat &x, const OriginMat &W, const OriginMat *b, std::pair<int, int> stride,
                      std::pair<int, int> pad, const char *who)
{
    if (unlikely(x.shape().size() != 4))
    {
        THROW_INVALID_ARG("{}: x must be 4D (N, C, H, W), but got shape {}", who, x.shape().to_string());
    }
    if (unlikely(W.shape().size() != 4))
    {
        THROW_INVALID_ARG("{}: W must be 4D (OC, C, KH, KW), but got shape {}", who, W.shape().to_string());
    }
    if (unlikely(x.shape()[1] != W.shape()[1]))
    {
        THROW_INVALID_ARG("{}: channel mismatch - x has {} channels, but W expects {} channels", who, x.shape()[1], W.shape()[1]);
    }
    if (unlikely(b != nullptr && b->elements() != W.shape()[0]))
    {
        THROW_INVALID_ARG("{}: bias must have {} elements, but got shape {}", who, W.shape()[0], b->shape().to_string());
    }
    VALIDATE_SAME_DTYPE(x, W);
    VALIDATE_SAME_CUDA_DEVICE(x, W);
    const ConvGeom g = conv_geom(x.shape(), {(int)W.shape()[2], (int)W.shape()[3]}, stride, pad, who);
    if (unlikely(!odl_conv_form(g, x.dtype())))
    {
        THROW_RUNTIME_ERROR("{}: the B200 backend takes float32 tensors with one stride and one padding for both image axes "
                            "(got dtype {}, stride=({},{}), pad=({},{}))",
                            who, dtype_to_string(x.dtype()), g.SH, g.SW, g.PH, g.PW);
    }
    return g;
}
}  // namespace

std::unique_ptr<Mat> conv2d(const OriginMat &x, const OriginMat &W, const OriginMat *b, std::pair<int, int> stride,
                            std::pair<int, int> pad)
{
    const ConvGeom g = conv_checked(x, W, b, stride, pad, "conv2d");
    std::unique_ptr<Mat> kx, kw, kb;
    const OriginMat &X = as_contiguous(x, kx);
    const OriginMat &F = as_contiguous(W, kw);
    const OriginMat *B = b ? &as_contiguous(*b, kb) : nullptr;
    const size_t OC    = W.shape()[0];
    auto y = std::make_unique<OriginMat>(Shape{(size_t)g.N, OC, (size_t)g.OH, (size_t)g.OW}, X.dtype(), X.device());
    odl_ready(X.device());
    odl_check(odl_conv2d_forward(X.data_ptr<float>(), F.data_ptr<float>(), B ? B->data_ptr<float>() : nullptr,
                                 y->data_ptr<float>(), g.N, g.C, g.H, g.W, (int64_t)OC, g.KH, g.KW, g.SH, g.PH, ODL_ACT_NONE,
                                 precision_mode(), nullptr),
              "conv2d");
    return y;
}

std::vector<std::unique_ptr<Mat>> conv2d_backward(const OriginMat &gy, const OriginMat &x, const OriginMat &W,
                                                  const OriginMat *b, std::pair<int, int> stride, std::pair<int, int> pad)
{
    if (unlikely(gy.shape().size() != 4))
    {
        THROW_INVALID_ARG("conv2d_backward: gy must be 4D (N, OC, OH, OW), but got shape {}", gy.shape().to_string());
    }
    const ConvGeom g = conv_checked(x, W, b, stride, pad, "conv2d_backward");
    const size_t OC  = W.shape()[0];
    if (unlikely(gy.shape() != Shape({(size_t)g.N, OC, (size_t)g.OH, (size_t)g.OW})))
    {
        THROW_INVALID_ARG("conv2d_backward: gy has shape {}, expected ({}, {}, {}, {})", gy.shape().to_string(), g.N, OC, g.OH, g.OW);
    }
    std::unique_ptr<Mat> kg, kx, kw;
    const OriginMat &G = as_contiguous(gy, kg);
    const OriginMat &X = as_contiguous(x, kx);
    const OriginMat &F = as_contiguous(W, kw);
    auto gx = std::make_unique<OriginMat>(X.shape(), X.dtype(), X.device());
    auto gw = std::make_unique<OriginMat>(F.shape(), F.dtype(), F.device());
    std::unique_ptr<OriginMat> gb;
    if (b != nullptr)
        gb = std::make_unique<OriginMat>(Shape{OC}, X.dtype(), X.device());
    odl_ready(X.device());
    odl_check(odl_conv2d_backward(G.data_ptr<float>(), X.data_ptr<float>(), F.data_ptr<float>(), gx->data_ptr<float>(),
                                  gw->data_ptr<float>(), gb ? gb->data_ptr<float>() : nullptr, g.N, g.C, g.H, g.W, (int64_t)OC,
                                  g.KH, g.KW, g.SH, g.PH, conv_gradient_layout(), precision_mode(), nullptr),
              "conv2d_backward");
    std::vector<std::unique_ptr<Mat>> grads;  // {gx, gW, [gb]}
    grads.push_back(std::move(gx));
    grads.push_back(std::move(gw));
    if (gb)
        grads.push_back(std::move(gb));
    return grads;
}

}  // namespace cuda
}  // namespace origin
