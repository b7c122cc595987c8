// Host orchestration of the fused entry points: Linear forward / backward and im2col Conv2d forward / backward on top
// of the tcgen05 GEMM, the operand-preparation pass and the conv helper kernels.  No arithmetic happens here.
#include <cuda_runtime.h>

#include "../../include/odl_b200.h"
#include "gemm_tc.cuh"
#include "host_util.h"
#include "internal.h"

namespace odl
{

namespace
{
inline size_t a256(size_t x)
{
    return (x + 255) & ~size_t(255);
}
inline int64_t pad4(int64_t x)
{
    return (x + 3) & ~int64_t(3);
}
// worst-case scratch gemm_dispatch may carve for one operand (padded copy + low part)
inline size_t operand_worst(int64_t rows, int64_t cols)
{
    return 2 * a256(static_cast<size_t>(rows) * pad4(cols) * 4);
}
}  // namespace

int linear_forward(const float *x, const float *x_small, const float *w, const float *w_small, const float *b, float *y,
                   float *y_small, int64_t M, int64_t N, int64_t K, int w_layout, int relu, int precision,
                   cudaStream_t stream)
{
    if (w_layout != ODL_W_OUT_IN && w_layout != ODL_W_IN_OUT)
    {
        set_last_error("linear: unknown weight layout %d", w_layout);
        return kInvalidArgument;
    }
    if (!x || !w || !y || M <= 0 || N <= 0 || K <= 0)
    {
        set_last_error("linear: invalid argument (M=%lld N=%lld K=%lld)", (long long)M, (long long)N, (long long)K);
        return kInvalidArgument;
    }
    int flags = 0;
    if (b)
        flags |= kEpiBias;
    if (relu)
        flags |= kEpiRelu;
    if (y_small)
        flags |= kEpiSmall;
    const int transB  = w_layout == ODL_W_OUT_IN ? 1 : 0;
    const int64_t ldw = w_layout == ODL_W_OUT_IN ? K : N;
    return gemm_dispatch(0, transB, M, N, K, x, x_small, K, w, w_small, ldw, y, y_small, N, b, nullptr, 0, nullptr,
                         flags, precision, stream, true);
}

int linear_backward(const float *x, const float *x_small, const float *w, const float *w_small, const float *dy, const float *dy_small,
                    const float *y, float *dx, float *dx_small, const float *dx_mask_src, float *dx_colsum, float *dw,
                    float *db, int64_t M, int64_t N, int64_t K, int w_layout, int precision, cudaStream_t stream,
                    cudaEvent_t dw_done)
{
    // dw_done (optional): the weight gradient is computed FIRST and the event recorded right behind its GEMM, so that a
    // caller can start reducing dW over the ranks while dX is still being computed.  Same GEMMs, same results.
    if (w_layout != ODL_W_OUT_IN && w_layout != ODL_W_IN_OUT)
    {
        set_last_error("linear_backward: unknown weight layout %d", w_layout);
        return kInvalidArgument;
    }
    if (!dy || M <= 0 || N <= 0 || K <= 0 || (dx && !w) || (dw && !x))
    {
        set_last_error("linear_backward: invalid argument (M=%lld N=%lld K=%lld)", (long long)M, (long long)N,
                       (long long)K);
        return kInvalidArgument;
    }
    if (!is_ready())
    {
        set_last_error("odl_init has not been called");
        return kNotInitialized;
    }
    const int terms      = precision == ODL_PRECISION_3XTF32 ? 3 : 1;
    const size_t mn      = a256(static_cast<size_t>(M) * N * 4);
    const bool need_g    = (y != nullptr);                  // masked copy of dy
    const bool need_gs   = (terms == 3) && (dx || dw) && !(dy_small && !need_g);  // low part of g
    arena_reset();
    // exact scratch: the masked copy / low part of dy, plus whatever the two GEMMs must stage for x and W
    // (g itself is either dy or an arena buffer with N % 4 == 0 handled by the GEMM's own staging)
    const int64_t ldw = w_layout == ODL_W_OUT_IN ? K : N;
    const int64_t wr  = w_layout == ODL_W_OUT_IN ? N : K;
    size_t need = (need_g ? mn : 0) + (need_gs ? mn : 0) + 2 * operand_scratch(dy, nullptr, N, M, N, terms);
    if (dx)
        need += operand_scratch(w, w_small, ldw, wr, ldw, terms);
    if (dw)
        need += operand_scratch(x, x_small, K, M, K, terms);
    int rc = arena_reserve(need);
    if (rc)
        return rc;
    const float *g  = dy;
    float *g_buf    = nullptr;
    const float *g_small_in = (dy_small && !need_g) ? dy_small : nullptr;
    float *g_small  = nullptr;
    if (need_g)
    {
        g_buf = static_cast<float *>(arena_alloc(static_cast<size_t>(M) * N * 4));
        g     = g_buf;
    }
    if (need_gs)
        g_small = static_cast<float *>(arena_alloc(static_cast<size_t>(M) * N * 4));
    if ((need_g && !g_buf) || (need_gs && !g_small))
        return kCudaError;
    const float *gs = g_small ? g_small : g_small_in;
    if (db)
        ODL_CUDA_TRY(cudaMemsetAsync(db, 0, static_cast<size_t>(N) * 4, stream));
    if (need_g || need_gs || db)
    {
        // one pass over dy: ReLU mask, low part for the two GEMMs, bias gradient
        rc = split_launch(dy, N, (int)M, (int)N, y, N, g_buf, g_small, N, db, stream);
        if (rc)
            return rc;
    }
    auto weight_gradient = [&]() -> int {
        int rc = kOk;
        if (dw)
        {
            if (w_layout == ODL_W_OUT_IN)  // dW[N,K] = g^T . x
                rc = gemm_dispatch(1, 0, N, K, M, g, gs, N, x, x_small, K, dw, nullptr, K, nullptr, nullptr, 0, nullptr,
                                   0, precision, stream, false);
            else  // dW{K,N} = x^T . g
                rc = gemm_dispatch(1, 0, K, N, M, x, x_small, K, g, gs, N, dw, nullptr, N, nullptr, nullptr, 0, nullptr,
                                   0, precision, stream, false);
            if (rc)
                return rc;
        }
        if (dw_done)
            ODL_CUDA_TRY(cudaEventRecord(dw_done, stream));
        return kOk;
    };
    if (dw_done && (rc = weight_gradient()))
        return rc;
    if (dx)
    {
        // dx[M,K] = g[M,N] . W   ([N,K]: B stored [reduce][out] -> transB = 0;  {K,N}: stored [out][reduce] -> 1)
        const int transB  = w_layout == ODL_W_OUT_IN ? 0 : 1;
        const int64_t ldw = w_layout == ODL_W_OUT_IN ? K : N;
        int flags         = 0;
        if (dx_small)
            flags |= kEpiSmall;
        if (dx_mask_src)
            flags |= kEpiMask;
        if (dx_colsum)
        {
            flags |= kEpiColsum;
            ODL_CUDA_TRY(cudaMemsetAsync(dx_colsum, 0, static_cast<size_t>(K) * 4, stream));
        }
        rc = gemm_dispatch(0, transB, M, K, N, g, gs, N, w, w_small, ldw, dx, dx_small, K, nullptr, dx_mask_src, K,
                           dx_colsum, flags, precision, stream, false);
        if (rc)
            return rc;
    }
    if (!dw_done && (rc = weight_gradient()))
        return rc;
    return kOk;
}

int conv2d_forward(const float *x, const float *w, const float *b, float *y, int64_t N, int64_t C, int64_t H, int64_t W,
                   int64_t OC, int KH, int KW, int S, int P, int act, int precision, cudaStream_t stream, const float *scale)
{
    if (!is_ready())
    {
        set_last_error("odl_init has not been called");
        return kNotInitialized;
    }
    if (!x || !w || !y || OC <= 0 || act < 0 || act > 2)
    {
        set_last_error("conv2d: null buffer or unknown activation %d", act);
        return kInvalidArgument;
    }
    const int OH = conv_out_size(H, KH, S, P), OW = conv_out_size(W, KW, S, P);
    if (OH <= 0 || OW <= 0)
    {
        set_last_error("conv2d: invalid output size OH=%d, OW=%d for input H=%lld, W=%lld", OH, OW, (long long)H,
                       (long long)W);
        return kInvalidArgument;
    }
    if (precision != ODL_PRECISION_3XTF32 && precision != ODL_PRECISION_TF32)
    {
        set_last_error("conv2d: unknown precision %d", precision);
        return kInvalidArgument;
    }
    const int terms     = precision == ODL_PRECISION_3XTF32 ? 3 : 1;
    const int64_t rows  = N * OH * OW;
    const int64_t ckk   = C * KH * KW;
    if (conv_fwd_direct_eligible(N, C, H, W, OC, KH, KW, OH, OW))
        return conv_fwd_direct_launch(x, w, b, scale, y, N, C, H, W, OC, KH, KW, S, P, OH, OW, act, stream);
    if (conv_igemm_eligible(N, C, H, W, OC, KH, KW, OH, OW))
    {
        // implicit GEMM: no column matrix; only the (small) weight matrix is prepared -- padded to a pitch of 4 floats
        // when needed and split into its 3xTF32 low part
        const int64_t ldw = pad4(ckk);
        const bool w_ok   = ldw == ckk && !(reinterpret_cast<uintptr_t>(w) & 15);
        const size_t wb   = a256(static_cast<size_t>(OC) * ldw * 4);
        arena_reset();
        int rc = arena_reserve(2 * wb);
        if (rc)
            return rc;
        float *w_big   = w_ok ? nullptr : static_cast<float *>(arena_alloc(wb));
        float *w_small = terms == 3 ? static_cast<float *>(arena_alloc(wb)) : nullptr;
        if ((!w_ok && !w_big) || (terms == 3 && !w_small))
            return kCudaError;
        if (w_big || w_small)
        {
            rc = split_launch(w, ckk, (int)OC, (int)ckk, nullptr, 0, w_big, w_small, ldw, nullptr, stream);
            if (rc)
                return rc;
        }
        return conv_igemm_launch(x, w_big ? w_big : w, w_small, ldw, b, scale, y, N, C, H, W, OC, KH, KW, S, P, OH, OW, act,
                                 terms, stream);
    }
    const int64_t ldcol = pad4(ckk);
    const size_t colb   = a256(static_cast<size_t>(rows) * ldcol * 4);
    arena_reset();
    int rc = arena_reserve(colb * (terms == 3 ? 2 : 1) + operand_worst(OC, ckk));
    if (rc)
        return rc;
    float *col   = static_cast<float *>(arena_alloc(colb));
    float *col_s = terms == 3 ? static_cast<float *>(arena_alloc(colb)) : nullptr;
    if (!col || (terms == 3 && !col_s))
        return kCudaError;
    rc = im2col_launch(x, col, col_s, N, C, H, W, KH, KW, S, P, stream);
    if (rc)
        return rc;
    int flags = kEpiNCHW;
    if (b)
        flags |= kEpiBias;
    if (act == 1)
        flags |= kEpiRelu;
    if (act == 2)
        flags |= kEpiSilu;
    if (scale)
        flags |= kEpiScale;
    // y_flat[rows, OC] = col[rows, ckk] . W[OC, ckk]^T, written straight into NCHW by the epilogue
    return gemm_dispatch(0, 1, rows, OC, ckk, col, col_s, ldcol, w, nullptr, ckk, y, nullptr, OC, b, nullptr, 0, nullptr, flags,
                         precision, stream, false, OH * OW, scale);
}

int conv2d_backward(const float *gy, const float *x, const float *w, float *gx, float *gw, float *gb, int64_t N, int64_t C,
                    int64_t H, int64_t W, int64_t OC, int KH, int KW, int S, int P, int mode, int precision,
                    cudaStream_t stream)
{
    if (!is_ready())
    {
        set_last_error("odl_init has not been called");
        return kNotInitialized;
    }
    if (!gy || (gw && !x) || (gx && !w) || OC <= 0 || (mode != 0 && mode != 1))
    {
        set_last_error("conv2d_backward: invalid argument");
        return kInvalidArgument;
    }
    const int OH = conv_out_size(H, KH, S, P), OW = conv_out_size(W, KW, S, P);
    if (OH <= 0 || OW <= 0)
    {
        set_last_error("conv2d_backward: invalid output size OH=%d, OW=%d", OH, OW);
        return kInvalidArgument;
    }
    const int terms     = precision == ODL_PRECISION_3XTF32 ? 3 : 1;
    const int64_t hw    = static_cast<int64_t>(OH) * OW;
    const int64_t rows  = N * hw;
    const int64_t ckk   = C * KH * KW;
    const int64_t ldcol = pad4(ckk);
    const int64_t ldg   = mode == 0 ? pad4(OC) : OC;
    const int64_t ldt   = pad4(rows);
    const size_t colb   = a256(static_cast<size_t>(rows) * ldcol * 4);
    const size_t gyb    = a256(static_cast<size_t>(rows) * pad4(OC) * 4);
    const size_t ctb    = a256(static_cast<size_t>(ckk) * ldt * 4);
    arena_reset();
    const bool dx_direct = gx && conv_dx_direct_eligible(N, C, H, W, OC, KH, KW, S);
    // weight gradient without a column matrix: for small layers a direct fp32 kernel (measured 0.188 / 0.095 / 0.041 ms
    // against 0.206 / 0.099 / 0.063 ms for the benchmark's first three conv layers), else the implicit GEMM over pixels
    // (the correct gradient layout only: gy must be a real, 16-byte-aligned NCHW tensor)
    const bool dw_igemm_ok = gw && mode == 0 && !(reinterpret_cast<uintptr_t>(gy) & 15) &&
                             conv_dw_igemm_eligible(N, C, H, W, OC, KH, KW, OH, OW);
    const bool dw_direct_ok = gw && conv_dw_direct_eligible(N, C, H, W, OC, KH, KW, OH, OW);
    const bool dw_direct = dw_direct_ok;
    const bool dw_igemm  = dw_igemm_ok && !dw_direct;
    // stride 1, the correct gradient layout: gx is itself a convolution of gy (no column-gradient matrix, no col2im)
    const bool dx_igemm = gx && !dx_direct && mode == 0 && conv_dx_igemm_eligible(N, C, H, W, OC, KH, KW, S, P, OH, OW);
    const size_t wfb    = a256(static_cast<size_t>(C) * pad4(OC * KH * KW) * 4);
    const size_t gysb = a256(static_cast<size_t>(rows) * OC * 4);
    const size_t slb  = dw_igemm ? a256(conv_dw_igemm_scratch(N, C, OC, KH, KW, OH, OW) * 4) : 0;
    int rc = arena_reserve((dx_igemm ? 2 * wfb : 0) + (dw_igemm ? gysb + slb : 0) +
                           (gw && !dw_direct && !dw_igemm ? colb * (terms == 3 ? 2 : 1) : 0) + 2 * gyb +
                           (gx && !dx_direct && !dx_igemm ? ctb : 0) + 2 * operand_worst(rows, OC) + operand_worst(OC, ckk));
    if (rc)
        return rc;
    // the direct weight-gradient kernel stages gy pixel by pixel and sums the bias gradient on the side (true layout only)
    const bool gb_with_dw = gb && dw_direct && mode == 0;
    if (gb && !gb_with_dw)
    {
        rc = channel_sum_launch(gy, gb, N, OC, hw, stream);
        if (rc)
            return rc;
    }
    // Input gradient of a conv with few products per output: direct fp32 kernel, no column-gradient matrix
    if (dx_direct)
    {
        rc = conv_dx_direct_launch(gy, w, gx, N, C, H, W, OC, KH, KW, S, P, OH, OW, mode, stream);
        if (rc)
            return rc;
        gx = nullptr;
    }
    if (dx_igemm)
    {
        float *wf   = static_cast<float *>(arena_alloc(wfb));
        float *wf_s = terms == 3 ? static_cast<float *>(arena_alloc(wfb)) : nullptr;
        if (!wf || (terms == 3 && !wf_s))
            return kCudaError;
        rc = conv_dx_igemm_launch(gy, w, wf, wf_s, gx, N, C, H, W, OC, KH, KW, P, OH, OW, terms, stream);
        if (rc)
            return rc;
        gx = nullptr;
    }
    // Weight gradient of a small conv: direct fp32 kernel, the column matrix only ever exists tile-wise in shared memory
    if (dw_direct)
    {
        // from image tiles in shared memory where a tile's window fits, else from gathered column blocks
        rc = conv_dw_tile_eligible(N, C, H, W, OC, KH, KW, S, P, OH, OW)
                 ? conv_dw_tile_launch(x, gy, gw, gb_with_dw ? gb : nullptr, N, C, H, W, OC, KH, KW, S, P, OH, OW, mode, stream)
                 : conv_dw_direct_launch(x, gy, gw, gb_with_dw ? gb : nullptr, N, C, H, W, OC, KH, KW, S, P, OH, OW, mode, stream);
        if (rc)
            return rc;
        gw = nullptr;
    }
    if (dw_igemm)
    {
        float *gys = terms == 3 ? static_cast<float *>(arena_alloc(gysb)) : nullptr;
        float *sl  = static_cast<float *>(arena_alloc(slb));
        if ((terms == 3 && !gys) || !sl)
            return kCudaError;
        if (gys)
        {
            rc = split_launch(gy, hw, (int)(N * OC), (int)hw, nullptr, 0, nullptr, gys, hw, nullptr, stream);
            if (rc)
                return rc;
        }
        rc = conv_dw_igemm_launch(x, gy, gys, sl, gw, N, C, H, W, OC, KH, KW, S, P, OH, OW, terms, stream);
        if (rc)
            return rc;
        gw = nullptr;
    }
    if (!gw && !gx)
        return kOk;
    // gy as a row matrix [rows, OC]: permuted copy (mode 0) or the reference's reinterpretation of the NCHW buffer
    const float *gyf   = gy;
    const float *gyf_s = nullptr;
    if (mode == 0)
    {
        float *t  = static_cast<float *>(arena_alloc(gyb));
        float *ts = terms == 3 ? static_cast<float *>(arena_alloc(gyb)) : nullptr;
        if (!t || (terms == 3 && !ts))
            return kCudaError;
        rc = nchw_to_rows_launch(gy, t, ts, N, OC, hw, ldg, stream);
        if (rc)
            return rc;
        gyf = t, gyf_s = ts;
    }
    if (gw)
    {
        float *col   = static_cast<float *>(arena_alloc(colb));
        float *col_s = terms == 3 ? static_cast<float *>(arena_alloc(colb)) : nullptr;
        if (!col || (terms == 3 && !col_s))
            return kCudaError;
        rc = im2col_launch(x, col, col_s, N, C, H, W, KH, KW, S, P, stream);
        if (rc)
            return rc;
        // gW[OC, ckk] = gyf^T . col   (reduction over rows: both operands MN-major; split-K inside the launcher)
        rc = gemm_dispatch(1, 0, OC, ckk, rows, gyf, gyf_s, ldg, col, col_s, ldcol, gw, nullptr, ckk, nullptr, nullptr, 0,
                           nullptr, 0, precision, stream, false);
        if (rc)
            return rc;
    }
    if (gx)
    {
        float *colT = static_cast<float *>(arena_alloc(ctb));
        if (!colT)
            return kCudaError;
        // colT[ckk, rows] = W^T[ckk, OC] . gyf^T[OC, rows]
        rc = gemm_dispatch(1, 1, ckk, rows, OC, w, nullptr, ckk, gyf, gyf_s, ldg, colT, nullptr, ldt, nullptr, nullptr, 0,
                           nullptr, 0, precision, stream, false);
        if (rc)
            return rc;
        rc = col2im_launch(colT, 1, ldt, gx, N, C, H, W, KH, KW, S, P, stream);
        if (rc)
            return rc;
    }
    return kOk;
}

}  // namespace odl
