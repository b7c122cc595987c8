// Input gradient of conv2d without the column matrix, for convolutions with few products per output element:
//
//   gx[n,c,h,w] = sum over the taps (kh, kw) that reach (h, w), ascending, of
//                 ( sum over oc, ascending, of gy_rows[(n,oh,ow), oc] * w[oc,c,kh,kw] ),   oh = (h+P-kh)/S, ow = (w+P-kw)/S
//
// which is the reference's conv2d_backward for x (src/mat/origin/cpu/conv/conv2d.cpp:534-600: gcol = gy_rows . W, then
// col2im) with the same summation order and fp32 rounding of every product and sum, so it agrees with the CPU
// restatement to the last bit -- and it is plain fp32, more accurate than the 3xTF32 GEMM it replaces.  The explicit path
// writes the 108 x 409600 column-gradient matrix of the first conv layer (177 MB) and reads it back; this kernel reads
// gy (L1 / L2 resident, reused by the KH*KW/S^2 taps) and writes gx once.  It runs on the CUDA cores: with
// OC * ceil(KH/S) * ceil(KW/S) products per output (144 for that layer) the work is 0.7 GFLOP, far below what the
// memory traffic of the GEMM path costs.  The launcher takes it up to 256 products per output (measured crossover:
// 576 products -- 64 -> 64 channels, 3 x 3 -- is 5 % slower than the GEMM path); above that the tensor-core GEMM +
// gather col2im path is used.
//
// One thread = one (n, h, w) position and CT consecutive input channels (the gy values it loads are shared by them);
// the weights of the channel group sit in shared memory as one float4 per (oc, kh, kw).  gy_layout 0: gy_rows is the permuted NCHW gradient (the true
// gradient); 1: the NCHW buffer reinterpreted as [N*OH*OW, OC] as the reference does.
#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/odl_b200.h"
#include "gemm_tc.cuh"
#include "host_util.h"
#include "internal.h"

namespace odl
{
extern int g_conv_mode;
namespace
{
struct DxGeom
{
    int N, C, H, W, OC, KH, KW, S, P, OH, OW;
};

template <int CT>
__global__ void __launch_bounds__(256) conv_dx_direct_kernel(const float *__restrict__ gy, const float *__restrict__ w,
                                                             float *__restrict__ gx, const DxGeom g, const int layout)
{
    extern __shared__ float4 ws[];  // [OC][KH][KW] x {the group's (up to 4) input channels}: one 128-bit read per product group
    const int c0  = blockIdx.y * CT;
    const int khw = g.KH * g.KW;
    for (int i = threadIdx.x; i < g.OC * khw; i += blockDim.x)
    {
        const int oc = i / khw, k = i - oc * khw;
        float v[4]   = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ct = 0; ct < CT; ++ct)
            if (c0 + ct < g.C)
                v[ct] = __ldg(w + (static_cast<int64_t>(oc) * g.C + c0 + ct) * khw + k);
        ws[i] = make_float4(v[0], v[1], v[2], v[3]);
    }
    __syncthreads();
    const int64_t total = static_cast<int64_t>(g.N) * g.H * g.W;
    const int64_t idx   = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total)
        return;
    const int wq = static_cast<int>(idx % g.W);
    const int t  = static_cast<int>(idx / g.W);
    const int hq = t % g.H;
    const int n  = t / g.H;
    const int ohw = g.OH * g.OW;
    float acc[CT];
#pragma unroll
    for (int ct = 0; ct < CT; ++ct)
        acc[ct] = 0.f;
    // only taps with (h + P - kh) and (w + P - kw) divisible by the stride contribute: walk those, ascending
    const int hp = hq + g.P, wp = wq + g.P;
    const int kh0 = hp % g.S, kw0 = wp % g.S;
    const int ow0 = (wp - kw0) / g.S;
    int oh        = (hp - kh0) / g.S;
    for (int kh = kh0; kh < g.KH && oh >= 0; kh += g.S, --oh)
    {
        if (oh >= g.OH)
            continue;
        int ow = ow0;
        for (int kw = kw0; kw < g.KW && ow >= 0; kw += g.S, --ow)
        {
            if (ow >= g.OW)
                continue;
            const int pix = oh * g.OW + ow;
            // element (row, oc) of gy_rows: layout 0 -> gy[n][oc][pix]; layout 1 -> flat[(n*ohw + pix) * OC + oc]
            const float *gp   = layout == 0 ? gy + static_cast<int64_t>(n) * g.OC * ohw + pix
                                            : gy + (static_cast<int64_t>(n) * ohw + pix) * g.OC;
            const int gstride = layout == 0 ? ohw : 1;
            const float4 *wp_ = ws + kh * g.KW + kw;
            float s[CT];
#pragma unroll
            for (int ct = 0; ct < CT; ++ct)
                s[ct] = 0.f;
#pragma unroll 4
            for (int oc = 0; oc < g.OC; ++oc)
            {
                const float gv  = __ldg(gp + static_cast<int64_t>(oc) * gstride);
                const float4 w4 = wp_[oc * khw];
                const float wv[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
                for (int ct = 0; ct < CT; ++ct)
                    s[ct] = __fadd_rn(s[ct], __fmul_rn(gv, wv[ct]));
            }
#pragma unroll
            for (int ct = 0; ct < CT; ++ct)
                acc[ct] = __fadd_rn(acc[ct], s[ct]);
        }
    }
#pragma unroll
    for (int ct = 0; ct < CT; ++ct)
        if (c0 + ct < g.C)
            gx[((static_cast<int64_t>(n) * g.C + c0 + ct) * g.H + hq) * g.W + wq] = acc[ct];
}

// The same sums with the channel count, the kernel size, the stride and the gradient layout fixed at compile time (the
// shapes of the reference's CNN): the tap loops unroll into ceil(KT/ST)^2 guarded blocks of OCT products each, the
// weight reads become constant offsets from one base, and in the row layout the OCT gradients of a tap arrive as
// 128-bit loads.  Same order of taps and of output channels, so the same bits as the generic kernel.
template <int CT, int OCT, int KT, int ST, int LAYOUT>
__global__ void __launch_bounds__(256) conv_dx_direct_fixed_kernel(const float *__restrict__ gy, const float *__restrict__ w,
                                                                   float *__restrict__ gx, const DxGeom g)
{
    constexpr int KHW = KT * KT;
    constexpr int T   = (KT + ST - 1) / ST;
    constexpr int C4 = (CT + 3) / 4;  // 128-bit weight words per (oc, tap): the group's channels, padded to a multiple of 4
    __shared__ float4 ws[OCT * KHW * C4];
    const int c0 = blockIdx.y * CT;
    for (int i = threadIdx.x; i < OCT * KHW; i += 256)
    {
        const int oc = i / KHW, k = i - oc * KHW;
        float v[4 * C4];
#pragma unroll
        for (int ct = 0; ct < 4 * C4; ++ct)
            v[ct] = (ct < CT && c0 + ct < g.C) ? __ldg(w + (static_cast<int64_t>(oc) * g.C + c0 + ct) * KHW + k) : 0.f;
#pragma unroll
        for (int q = 0; q < C4; ++q)
            ws[i * C4 + q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
    }
    __syncthreads();
    const int64_t total = static_cast<int64_t>(g.N) * g.H * g.W;
    const int64_t idx   = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total)
        return;
    const int wq  = static_cast<int>(idx % g.W);
    const int t_  = static_cast<int>(idx / g.W);
    const int hq  = t_ % g.H;
    const int n   = t_ / g.H;
    const int ohw = g.OH * g.OW;
    float acc[CT];
#pragma unroll
    for (int ct = 0; ct < CT; ++ct)
        acc[ct] = 0.f;
    const int hp = hq + g.P, wp = wq + g.P;
    const int kh0 = hp % ST, kw0 = wp % ST;
    const int oh0 = hp / ST, ow0 = wp / ST;
    const float *gn = LAYOUT == 0 ? gy + static_cast<int64_t>(n) * OCT * ohw : gy + static_cast<int64_t>(n) * ohw * OCT;
#pragma unroll
    for (int t = 0; t < T; ++t)
    {
        const int kh = kh0 + t * ST, oh = oh0 - t;
        if ((KT % ST != 0 && kh >= KT) || static_cast<unsigned>(oh) >= static_cast<unsigned>(g.OH))
            continue;
#pragma unroll
        for (int u = 0; u < T; ++u)
        {
            const int kw = kw0 + u * ST, ow = ow0 - u;
            if ((KT % ST != 0 && kw >= KT) || static_cast<unsigned>(ow) >= static_cast<unsigned>(g.OW))
                continue;
            const int pix     = oh * g.OW + ow;
            const float4 *wt  = ws + (kh * KT + kw) * C4;
            float gv[OCT];
            if (LAYOUT == 0)
            {
                const float *gp = gn + pix;
#pragma unroll
                for (int oc = 0; oc < OCT; ++oc)
                    gv[oc] = __ldg(gp + oc * ohw);
            }
            else
            {
                const float4 *gp = reinterpret_cast<const float4 *>(gn + static_cast<int64_t>(pix) * OCT);
#pragma unroll
                for (int q = 0; q < OCT / 4; ++q)
                {
                    const float4 v = __ldg(gp + q);
                    gv[4 * q] = v.x, gv[4 * q + 1] = v.y, gv[4 * q + 2] = v.z, gv[4 * q + 3] = v.w;
                }
            }
            float s[CT];
#pragma unroll
            for (int ct = 0; ct < CT; ++ct)
                s[ct] = 0.f;
#pragma unroll
            for (int oc = 0; oc < OCT; ++oc)
            {
                float wv[4 * C4];
#pragma unroll
                for (int q = 0; q < C4; ++q)
                {
                    const float4 w4 = wt[oc * KHW * C4 + q];
                    wv[4 * q] = w4.x, wv[4 * q + 1] = w4.y, wv[4 * q + 2] = w4.z, wv[4 * q + 3] = w4.w;
                }
#pragma unroll
                for (int ct = 0; ct < CT; ++ct)
                    s[ct] = __fadd_rn(s[ct], __fmul_rn(gv[oc], wv[ct]));
            }
#pragma unroll
            for (int ct = 0; ct < CT; ++ct)
                acc[ct] = __fadd_rn(acc[ct], s[ct]);
        }
    }
#pragma unroll
    for (int ct = 0; ct < CT; ++ct)
        if (c0 + ct < g.C)
            gx[((static_cast<int64_t>(n) * g.C + c0 + ct) * g.H + hq) * g.W + wq] = acc[ct];
}

// Two positions per thread, (h, w) and (h, w + ST): they meet the same taps (kh, kw) -- one weight read serves both -- at
// output columns ow and ow + 1, so the second position's gradients sit right behind the first's.  Needs W to be a
// multiple of 2 * ST.  Thread j of a row takes w = (j / ST) * 2 * ST + j % ST.
template <int CT, int OCT, int KT, int ST, int LAYOUT>
__global__ void __launch_bounds__(256) conv_dx_direct_pair_kernel(const float *__restrict__ gy, const float *__restrict__ w,
                                                                  float *__restrict__ gx, const DxGeom g)
{
    constexpr int KHW = KT * KT;
    constexpr int T   = (KT + ST - 1) / ST;
    constexpr int C4 = (CT + 3) / 4;  // 128-bit weight words per (oc, tap): the group's channels, padded to a multiple of 4
    __shared__ float4 ws[OCT * KHW * C4];
    const int c0 = blockIdx.y * CT;
    for (int i = threadIdx.x; i < OCT * KHW; i += 256)
    {
        const int oc = i / KHW, k = i - oc * KHW;
        float v[4 * C4];
#pragma unroll
        for (int ct = 0; ct < 4 * C4; ++ct)
            v[ct] = (ct < CT && c0 + ct < g.C) ? __ldg(w + (static_cast<int64_t>(oc) * g.C + c0 + ct) * KHW + k) : 0.f;
#pragma unroll
        for (int q = 0; q < C4; ++q)
            ws[i * C4 + q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
    }
    __syncthreads();
    const int half      = g.W / 2;
    const int64_t total = static_cast<int64_t>(g.N) * g.H * half;
    const int64_t idx   = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total)
        return;
    const int j   = static_cast<int>(idx % half);
    const int t_  = static_cast<int>(idx / half);
    const int hq  = t_ % g.H;
    const int n   = t_ / g.H;
    const int wq  = (j / ST) * 2 * ST + j % ST;
    const int ohw = g.OH * g.OW;
    float acc[2][CT];
#pragma unroll
    for (int ct = 0; ct < CT; ++ct)
        acc[0][ct] = acc[1][ct] = 0.f;
    const int hp = hq + g.P, wp = wq + g.P;
    const int kh0 = hp % ST, kw0 = wp % ST;
    const int oh0 = hp / ST, ow0 = wp / ST;
    const float *gn = LAYOUT == 0 ? gy + static_cast<int64_t>(n) * OCT * ohw : gy + static_cast<int64_t>(n) * ohw * OCT;
#pragma unroll
    for (int t = 0; t < T; ++t)
    {
        const int kh = kh0 + t * ST, oh = oh0 - t;
        if ((KT % ST != 0 && kh >= KT) || static_cast<unsigned>(oh) >= static_cast<unsigned>(g.OH))
            continue;
#pragma unroll
        for (int u = 0; u < T; ++u)
        {
            const int kw = kw0 + u * ST, ow = ow0 - u;
            if (KT % ST != 0 && kw >= KT)
                continue;
            const bool va = static_cast<unsigned>(ow) < static_cast<unsigned>(g.OW);
            const bool vb = static_cast<unsigned>(ow + 1) < static_cast<unsigned>(g.OW);
            if (!va && !vb)
                continue;
            const int pix    = oh * g.OW + ow;
            const float4 *wt = ws + (kh * KT + kw) * C4;
            float ga[OCT], gb[OCT];
            if (LAYOUT == 0)
            {
                const float *gp = gn + pix;
#pragma unroll
                for (int oc = 0; oc < OCT; ++oc)
                {
                    ga[oc] = va ? __ldg(gp + oc * ohw) : 0.f;
                    gb[oc] = vb ? __ldg(gp + oc * ohw + 1) : 0.f;
                }
            }
            else
            {
                const float4 *gp = reinterpret_cast<const float4 *>(gn + static_cast<int64_t>(pix) * OCT);
#pragma unroll
                for (int q = 0; q < OCT / 4; ++q)
                {
                    const float4 a = va ? __ldg(gp + q) : make_float4(0.f, 0.f, 0.f, 0.f);
                    const float4 b = vb ? __ldg(gp + OCT / 4 + q) : make_float4(0.f, 0.f, 0.f, 0.f);
                    ga[4 * q] = a.x, ga[4 * q + 1] = a.y, ga[4 * q + 2] = a.z, ga[4 * q + 3] = a.w;
                    gb[4 * q] = b.x, gb[4 * q + 1] = b.y, gb[4 * q + 2] = b.z, gb[4 * q + 3] = b.w;
                }
            }
            float sa[CT], sb[CT];
#pragma unroll
            for (int ct = 0; ct < CT; ++ct)
                sa[ct] = sb[ct] = 0.f;
#pragma unroll
            for (int oc = 0; oc < OCT; ++oc)
            {
                float wv[4 * C4];
#pragma unroll
                for (int q = 0; q < C4; ++q)
                {
                    const float4 w4 = wt[oc * KHW * C4 + q];
                    wv[4 * q] = w4.x, wv[4 * q + 1] = w4.y, wv[4 * q + 2] = w4.z, wv[4 * q + 3] = w4.w;
                }
#pragma unroll
                for (int ct = 0; ct < CT; ++ct)
                {
                    sa[ct] = __fadd_rn(sa[ct], __fmul_rn(ga[oc], wv[ct]));
                    sb[ct] = __fadd_rn(sb[ct], __fmul_rn(gb[oc], wv[ct]));
                }
            }
            // a tap outside the output for one of the two positions is skipped for it, as the reference's col2im does
#pragma unroll
            for (int ct = 0; ct < CT; ++ct)
            {
                if (va)
                    acc[0][ct] = __fadd_rn(acc[0][ct], sa[ct]);
                if (vb)
                    acc[1][ct] = __fadd_rn(acc[1][ct], sb[ct]);
            }
        }
    }
#pragma unroll
    for (int ct = 0; ct < CT; ++ct)
        if (c0 + ct < g.C)
        {
            float *dst = gx + ((static_cast<int64_t>(n) * g.C + c0 + ct) * g.H + hq) * g.W + wq;
            dst[0]     = acc[0][ct];
            dst[ST]    = acc[1][ct];
        }
}

template <int CT, int OCT, int KT, int ST>
int launch_dx_fixed(const float *gy, const float *w, float *gx, const DxGeom &g, int layout, cudaStream_t stream)
{
    const bool pair     = g.W % (2 * ST) == 0 && g_conv_mode != 5;  // test hook: conv mode 5 keeps one position per thread
    const int64_t total = static_cast<int64_t>(g.N) * g.H * (pair ? g.W / 2 : g.W);
    dim3 grid(static_cast<unsigned>((total + 255) / 256), static_cast<unsigned>((g.C + CT - 1) / CT));
    if (pair && layout == 0)
        conv_dx_direct_pair_kernel<CT, OCT, KT, ST, 0><<<grid, 256, 0, stream>>>(gy, w, gx, g);
    else if (pair)
        conv_dx_direct_pair_kernel<CT, OCT, KT, ST, 1><<<grid, 256, 0, stream>>>(gy, w, gx, g);
    else if (layout == 0)
        conv_dx_direct_fixed_kernel<CT, OCT, KT, ST, 0><<<grid, 256, 0, stream>>>(gy, w, gx, g);
    else
        conv_dx_direct_fixed_kernel<CT, OCT, KT, ST, 1><<<grid, 256, 0, stream>>>(gy, w, gx, g);
    ++g_launch_count;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
    {
        set_last_error("conv_dx_direct_fixed_kernel<%d,%d,%d,%d> launch failed: %s", CT, OCT, KT, ST, cudaGetErrorString(e));
        return kCudaError;
    }
    return kOk;
}

template <int CT>
int launch_dx(const float *gy, const float *w, float *gx, const DxGeom &g, int layout, cudaStream_t stream)
{
    const size_t smem   = sizeof(float4) * g.OC * g.KH * g.KW;
    const int64_t total = static_cast<int64_t>(g.N) * g.H * g.W;
    dim3 grid(static_cast<unsigned>((total + 255) / 256), static_cast<unsigned>((g.C + CT - 1) / CT));
    conv_dx_direct_kernel<CT><<<grid, 256, smem, stream>>>(gy, w, gx, g, layout);
    ++g_launch_count;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
    {
        set_last_error("conv_dx_direct_kernel<%d> launch failed: %s", CT, cudaGetErrorString(e));
        return kCudaError;
    }
    return kOk;
}

// Input channels per thread: up to 4 (one float4 of weights per (oc, kh, kw)); 0 when the weights of a group would not
// fit the default 48 KB of shared memory.
int channel_group(int64_t C, int64_t OC, int KH, int KW)
{
    if (OC * KH * KW * 16 > 48 * 1024)
        return 0;
    return C >= 4 ? 4 : static_cast<int>(C);
}
}  // namespace

bool conv_dx_direct_eligible(int64_t N, int64_t C, int64_t H, int64_t W, int64_t OC, int KH, int KW, int S)
{
    const int64_t products = OC * ((KH + S - 1) / S) * ((KW + S - 1) / S);
    return g_conv_mode != 1 && products <= 256 && channel_group(C, OC, KH, KW) > 0 && (N * H * W + 255) / 256 < (int64_t(1) << 31) &&
           (C + 3) / 4 <= 65535 && OC * KH * KW < (int64_t(1) << 24);
}

int conv_dx_direct_launch(const float *gy, const float *w, float *gx, int64_t N, int64_t C, int64_t H, int64_t W, int64_t OC,
                          int KH, int KW, int S, int P, int OH, int OW, int layout, cudaStream_t stream)
{
    DxGeom g;
    g.N = (int)N, g.C = (int)C, g.H = (int)H, g.W = (int)W, g.OC = (int)OC, g.KH = KH, g.KW = KW, g.S = S, g.P = P;
    g.OH = OH, g.OW = OW;
    // the compile-time shapes (test hook: conv mode 4 keeps the generic kernel); the row layout reads gy 16 bytes at a time
    const int ct = channel_group(C, OC, KH, KW);
    if (g_conv_mode != 4 && KH == KW && (layout == 0 || reinterpret_cast<uintptr_t>(gy) % 16 == 0))
    {
        if (ct == 3 && OC == 16 && KH == 6 && S == 2)
            return launch_dx_fixed<3, 16, 6, 2>(gy, w, gx, g, layout, stream);
        // eight input channels per thread where there are that many: half the gradient loads per product (the first-level
        // cache's load rate, not arithmetic, bounds the 16 -> 32 channel layer with four)
        const bool eight = C >= 8 && g_conv_mode != 8;  // test hook: conv mode 8 keeps four channels per thread
        if (ct == 4 && OC == 32 && KH == 3 && S == 2)
            return eight ? launch_dx_fixed<8, 32, 3, 2>(gy, w, gx, g, layout, stream)
                         : launch_dx_fixed<4, 32, 3, 2>(gy, w, gx, g, layout, stream);
        if (ct == 4 && OC == 32 && KH == 1 && S == 1)
            return eight ? launch_dx_fixed<8, 32, 1, 1>(gy, w, gx, g, layout, stream)
                         : launch_dx_fixed<4, 32, 1, 1>(gy, w, gx, g, layout, stream);
        if (ct == 4 && OC == 16 && KH == 3 && S == 1)
            return eight ? launch_dx_fixed<8, 16, 3, 1>(gy, w, gx, g, layout, stream)
                         : launch_dx_fixed<4, 16, 3, 1>(gy, w, gx, g, layout, stream);
        if (ct == 4 && OC == 16 && KH == 3 && S == 2)
            return eight ? launch_dx_fixed<8, 16, 3, 2>(gy, w, gx, g, layout, stream)
                         : launch_dx_fixed<4, 16, 3, 2>(gy, w, gx, g, layout, stream);
    }
    switch (ct)
    {
        case 4:
            return launch_dx<4>(gy, w, gx, g, layout, stream);
        case 3:
            return launch_dx<3>(gy, w, gx, g, layout, stream);
        case 2:
            return launch_dx<2>(gy, w, gx, g, layout, stream);
        case 1:
            return launch_dx<1>(gy, w, gx, g, layout, stream);
        default:
            set_last_error("conv_dx_direct: weights of one channel do not fit shared memory");
            return kTooLarge;
    }
}

}  // namespace odl
