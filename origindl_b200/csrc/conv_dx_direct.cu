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

extern int g_conv_mode;

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
    switch (channel_group(C, OC, KH, KW))
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
