// Forward conv2d on the CUDA cores, for layers with few output channels and a short reduction:
//
//   y[n,oc,oh,ow] = act( scale[oc] * sum over (c, kh, kw) ascending of x[n,c,oh*S-P+kh,ow*S-P+kw] * w[oc,c,kh,kw] + b[oc] )
//
// i.e. cuda::conv2d of the reference (src/mat/origin/cuda/conv/conv2d.cu:563-678: pad copy, im2col, matmul, broadcast
// bias add, NHWC -> NCHW copy) in one pass with no column matrix.  The first layers of the reference's CNNs have 3-32
// channels: as a GEMM they are [pixels] x [C*KH*KW <= 256] x [OC <= 32], a shape on which the tensor-core path spends
// its time gathering operands into shared memory for MMAs that use a sixteenth of the tensor core's width (the
// implicit-GEMM kernel needs 0.16 ms for the 3 -> 16, 6 x 6, stride 2 layer on 16 x 320 x 320, whose ideal traffic is
// 46 MB = 7 us).  Here one thread owns one output pixel and ALL its output channels: every input value it loads feeds OC
// fused multiply-adds whose weights come out of shared memory as broadcast 128-bit reads, consecutive lanes own
// consecutive ow so the loads of a tap and the NCHW stores of a channel are coalesced, and the arithmetic is plain fp32
// (one accumulator per output, k ascending -- the reference's order; no TF32 split involved, so it is more accurate than
// the tensor-core path it replaces).  0.7 GFLOP for that layer is FMA-issue bound at a few tens of microseconds.
#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/odl_b200.h"
#include "gemm_tc.cuh"
#include "host_util.h"
#include "internal.h"

namespace odl
{
namespace
{
struct FwdGeom
{
    int N, C, H, W, OC, KH, KW, S, P, OH, OW, ckk;
};

// OCT: output channels per thread (OC padded up with zero weights); KWT: kernel width, ST: stride, both known at compile
// time.  A thread owns TWO horizontally adjacent output pixels: the KWT + ST input values of a kernel row are loaded once
// (for stride < KWT the two windows overlap) and every 128-bit weight read out of shared memory feeds eight
// multiply-adds instead of four -- the kernel is bound by instruction issue, so fewer loads per FMA is what counts.
template <int OCT, int KWT, int ST>
__global__ void __launch_bounds__(256) conv_fwd_direct2_kernel(const float *__restrict__ x, const float *__restrict__ w,
                                                               const float *__restrict__ bias, const float *__restrict__ scale,
                                                               float *__restrict__ y, const FwdGeom g, const int act)
{
    extern __shared__ float4 ws4[];  // [ckk][OCT] weights, output channels beyond OC are zero
    float *ws = reinterpret_cast<float *>(ws4);
    for (int i = threadIdx.x; i < g.ckk * OCT; i += blockDim.x)
    {
        const int k = i / OCT, oc = i - k * OCT;
        ws[i]       = oc < g.OC ? __ldg(w + static_cast<int64_t>(oc) * g.ckk + k) : 0.f;
    }
    __syncthreads();
    const int pairs_w   = (g.OW + 1) >> 1;  // pixel pairs per output row
    const int64_t total = static_cast<int64_t>(g.N) * g.OH * pairs_w;
    const int64_t idx   = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total)
        return;
    const int ow = 2 * static_cast<int>(idx % pairs_w);
    const int t  = static_cast<int>(idx / pairs_w);
    const int oh = t % g.OH, n = t / g.OH;
    const bool second = ow + 1 < g.OW;
    const int h0 = oh * g.S - g.P, w0 = ow * g.S - g.P;
    constexpr int NV = KWT + ST;  // input values of one kernel row that the two windows cover together
    const bool cols_inside = w0 >= 0 && w0 + NV <= g.W;
    float acc0[OCT], acc1[OCT];
#pragma unroll
    for (int i = 0; i < OCT; ++i)
        acc0[i] = acc1[i] = 0.f;
    const float *xn = x + static_cast<int64_t>(n) * g.C * g.H * g.W;
    int k           = 0;
    for (int c = 0; c < g.C; ++c)
    {
        const float *xc = xn + static_cast<int64_t>(c) * g.H * g.W;
        for (int kh = 0; kh < g.KH; ++kh, k += KWT)
        {
            const int hh = h0 + kh;
            if (hh < 0 || hh >= g.H)
                continue;  // a row of taps outside the image adds nothing
            const float *xr = xc + static_cast<int64_t>(hh) * g.W + w0;
            float v[NV];
            if (cols_inside)
            {
#pragma unroll
                for (int i = 0; i < NV; ++i)
                    v[i] = __ldg(xr + i);
            }
            else
            {
#pragma unroll
                for (int i = 0; i < NV; ++i)
                    v[i] = (w0 + i >= 0 && w0 + i < g.W) ? __ldg(xr + i) : 0.f;
            }
#pragma unroll
            for (int kw = 0; kw < KWT; ++kw)
            {
                const float4 *wk = ws4 + (k + kw) * (OCT / 4);
                const float a = v[kw], b = v[kw + ST];
#pragma unroll
                for (int j = 0; j < OCT / 4; ++j)
                {
                    const float4 q  = wk[j];
                    acc0[4 * j]     = fmaf(a, q.x, acc0[4 * j]);
                    acc0[4 * j + 1] = fmaf(a, q.y, acc0[4 * j + 1]);
                    acc0[4 * j + 2] = fmaf(a, q.z, acc0[4 * j + 2]);
                    acc0[4 * j + 3] = fmaf(a, q.w, acc0[4 * j + 3]);
                    acc1[4 * j]     = fmaf(b, q.x, acc1[4 * j]);
                    acc1[4 * j + 1] = fmaf(b, q.y, acc1[4 * j + 1]);
                    acc1[4 * j + 2] = fmaf(b, q.z, acc1[4 * j + 2]);
                    acc1[4 * j + 3] = fmaf(b, q.w, acc1[4 * j + 3]);
                }
            }
        }
    }
    float *yp = y + (static_cast<int64_t>(n) * g.OC * g.OH + oh) * g.OW + ow;
    const int64_t plane = static_cast<int64_t>(g.OH) * g.OW;
    auto finish = [&](float v, int oc) {
        if (scale)
            v = __fmul_rn(v, __ldg(scale + oc));
        if (bias)
            v = __fadd_rn(v, __ldg(bias + oc));
        if (act == ODL_ACT_RELU)
            v = v > 0.f ? v : 0.f;
        else if (act == ODL_ACT_SILU)
            v = __fmul_rn(v, __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-v))));
        return v;
    };
#pragma unroll
    for (int oc = 0; oc < OCT; ++oc)
    {
        if (oc < g.OC)
        {
            yp[oc * plane] = finish(acc0[oc], oc);
            if (second)
                yp[oc * plane + 1] = finish(acc1[oc], oc);
        }
    }
}

// The general form: one pixel per thread, any kernel width and stride.  KWT > 0: kernel width known at compile time (the
// taps of a kernel row are then loaded together before their multiply-adds).
template <int OCT, int KWT>
__global__ void __launch_bounds__(256) conv_fwd_direct_kernel(const float *__restrict__ x, const float *__restrict__ w,
                                                              const float *__restrict__ bias, const float *__restrict__ scale,
                                                              float *__restrict__ y, const FwdGeom g, const int act)
{
    extern __shared__ float4 ws4[];  // [ckk][OCT] weights, output channels beyond OC are zero
    float *ws = reinterpret_cast<float *>(ws4);
    for (int i = threadIdx.x; i < g.ckk * OCT; i += blockDim.x)
    {
        const int k = i / OCT, oc = i - k * OCT;
        ws[i]       = oc < g.OC ? __ldg(w + static_cast<int64_t>(oc) * g.ckk + k) : 0.f;
    }
    __syncthreads();
    const int64_t total = static_cast<int64_t>(g.N) * g.OH * g.OW;
    const int64_t idx   = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total)
        return;
    const int ow = static_cast<int>(idx % g.OW);
    const int t  = static_cast<int>(idx / g.OW);
    const int oh = t % g.OH, n = t / g.OH;
    const int h0 = oh * g.S - g.P, w0 = ow * g.S - g.P;
    const int KW = KWT > 0 ? KWT : g.KW;
    const bool cols_inside = w0 >= 0 && w0 + KW <= g.W;  // no tap of a row falls left or right of the image
    float acc[OCT];
#pragma unroll
    for (int i = 0; i < OCT; ++i)
        acc[i] = 0.f;
    auto mac = [&](float v, int k) {
        const float4 *wk = ws4 + k * (OCT / 4);
#pragma unroll
        for (int j = 0; j < OCT / 4; ++j)
        {
            const float4 q = wk[j];
            acc[4 * j]     = fmaf(v, q.x, acc[4 * j]);
            acc[4 * j + 1] = fmaf(v, q.y, acc[4 * j + 1]);
            acc[4 * j + 2] = fmaf(v, q.z, acc[4 * j + 2]);
            acc[4 * j + 3] = fmaf(v, q.w, acc[4 * j + 3]);
        }
    };
    const float *xn = x + static_cast<int64_t>(n) * g.C * g.H * g.W;
    int k           = 0;
    for (int c = 0; c < g.C; ++c)
    {
        const float *xc = xn + static_cast<int64_t>(c) * g.H * g.W;
        for (int kh = 0; kh < g.KH; ++kh, k += KW)
        {
            const int hh = h0 + kh;
            if (hh < 0 || hh >= g.H)
                continue;  // a row of taps outside the image adds nothing
            const float *xr = xc + static_cast<int64_t>(hh) * g.W + w0;
            if (KWT > 0)
            {
                float v[KWT > 0 ? KWT : 1];
                if (cols_inside)
                {
#pragma unroll
                    for (int kw = 0; kw < KWT; ++kw)
                        v[kw] = __ldg(xr + kw);
                }
                else
                {
#pragma unroll
                    for (int kw = 0; kw < KWT; ++kw)
                        v[kw] = (w0 + kw >= 0 && w0 + kw < g.W) ? __ldg(xr + kw) : 0.f;
                }
#pragma unroll
                for (int kw = 0; kw < KWT; ++kw)
                    mac(v[kw], k + kw);
            }
            else
            {
                for (int kw = 0; kw < KW; ++kw)
                    mac((w0 + kw >= 0 && w0 + kw < g.W) ? __ldg(xr + kw) : 0.f, k + kw);
            }
        }
    }
    // epilogue in the order of the GEMM path: folded BatchNorm scale, bias, ReLU, SiLU; lanes = consecutive ow
    float *yp = y + (static_cast<int64_t>(n) * g.OC * g.OH + oh) * g.OW + ow;
    const int64_t plane = static_cast<int64_t>(g.OH) * g.OW;
#pragma unroll
    for (int oc = 0; oc < OCT; ++oc)
    {
        if (oc < g.OC)
        {
            float v = acc[oc];
            if (scale)
                v = __fmul_rn(v, __ldg(scale + oc));
            if (bias)
                v = __fadd_rn(v, __ldg(bias + oc));
            if (act == ODL_ACT_RELU)
                v = v > 0.f ? v : 0.f;
            else if (act == ODL_ACT_SILU)
                v = __fmul_rn(v, __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-v))));
            yp[oc * plane] = v;
        }
    }
}

template <int OCT>
void launch_fwd(int kw, int stride, size_t smem, cudaStream_t stream, const float *x, const float *w, const float *bias,
                const float *scale, float *y, const FwdGeom &g, int act)
{
    const int64_t pixels = static_cast<int64_t>(g.N) * g.OH * g.OW;
    const int64_t pairs  = static_cast<int64_t>(g.N) * g.OH * ((g.OW + 1) >> 1);
    const unsigned grid1 = static_cast<unsigned>((pixels + 255) / 256), grid2 = static_cast<unsigned>((pairs + 255) / 256);
    // (the pixel-pair form pays with 16 channels per thread; with 32 it holds 64 accumulators and measured slower)
#define ODL_FWD2(K, S_)                                                                                              \
    if (OCT == 16 && kw == K && stride == S_)                                                                        \
    {                                                                                                                \
        conv_fwd_direct2_kernel<OCT, K, S_><<<grid2, 256, smem, stream>>>(x, w, bias, scale, y, g, act);             \
        return;                                                                                                      \
    }
    ODL_FWD2(1, 1) ODL_FWD2(3, 1) ODL_FWD2(3, 2) ODL_FWD2(5, 1) ODL_FWD2(5, 2) ODL_FWD2(6, 2) ODL_FWD2(7, 2)
#undef ODL_FWD2
    switch (kw)
    {
        case 1: conv_fwd_direct_kernel<OCT, 1><<<grid1, 256, smem, stream>>>(x, w, bias, scale, y, g, act); break;
        case 3: conv_fwd_direct_kernel<OCT, 3><<<grid1, 256, smem, stream>>>(x, w, bias, scale, y, g, act); break;
        case 5: conv_fwd_direct_kernel<OCT, 5><<<grid1, 256, smem, stream>>>(x, w, bias, scale, y, g, act); break;
        default: conv_fwd_direct_kernel<OCT, 0><<<grid1, 256, smem, stream>>>(x, w, bias, scale, y, g, act); break;
    }
}
}  // namespace

extern int g_conv_mode;

// Layers this kernel takes: at most 32 output channels and a reduction of at most 256 (32 KB of weights in shared memory).
bool conv_fwd_direct_eligible(int64_t N, int64_t C, int64_t H, int64_t W, int64_t OC, int KH, int KW, int OH, int OW)
{
    return g_conv_mode != 1 && g_conv_mode != 3 && OC <= 32 && C * KH * KW <= 256 && N * C * H * W < (int64_t(1) << 31) &&
           N * OC * OH * OW < (int64_t(1) << 31);
}

int conv_fwd_direct_launch(const float *x, const float *w, const float *bias, const float *scale, float *y, int64_t N,
                           int64_t C, int64_t H, int64_t W, int64_t OC, int KH, int KW, int S, int P, int OH, int OW, int act,
                           cudaStream_t stream)
{
    FwdGeom g{(int)N, (int)C, (int)H, (int)W, (int)OC, KH, KW, S, P, OH, OW, (int)(C * KH * KW)};
    if (OC <= 16)
        launch_fwd<16>(KW, S, g.ckk * 16 * sizeof(float), stream, x, w, bias, scale, y, g, act);
    else
        launch_fwd<32>(KW, S, g.ckk * 32 * sizeof(float), stream, x, w, bias, scale, y, g, act);
    ++g_launch_count;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
    {
        set_last_error("conv_fwd_direct_kernel launch failed: %s", cudaGetErrorString(e));
        return kCudaError;
    }
    return kOk;
}

}  // namespace odl
