// Weight gradient of conv2d without a column matrix in HBM, for small convolutions (OC <= 32, C*KH*KW <= 256):
//
//   gw[oc, k] = sum over output pixels r of gy_rows[r, oc] * col[r, k],   col[r, (c,kh,kw)] = x[n, c, oh*S+kh-P, ow*S+kw-P]
//
// (the reference's conv2d_backward for W, src/mat/origin/cpu/conv/conv2d.cpp:534-600: im2col, then gy_rows^T . col).  The
// explicit path writes col and its 3xTF32 low part to HBM (2 x 177 MB for the first conv layer of the reference's CNN),
// reads them back in a split-K GEMM whose 16 x 108 output uses a fraction of one tensor-core tile, and needs gy
// re-laid out as rows.  Here a block stages PIX pixels of gy and of col in shared memory (col gathered from x through a
// per-block table k -> offset, like the implicit-GEMM forward) and every thread keeps a 4 x KT register tile of
// (oc, k) sums in plain fp32 FMAs; blocks walk the pixels grid-stride, store their partial gw into their own slice of
// a scratch buffer, and a second pass adds the slices in a fixed order (same bits every run).  The work is N*OH*OW * OC * C*KH*KW FMAs (0.7 G for that layer) on the CUDA cores.
//
// gy_layout 0: gy_rows is the permuted NCHW gradient (the true gradient); 1: the NCHW buffer reinterpreted as
// [N*OH*OW, OC] as the reference does.  Summation order differs from the reference's single accumulator (as it does in
// the split-K GEMM path): tolerance 1e-5, not bit-exactness.
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
struct DwGeom
{
    int N, C, H, W, OC, KH, KW, S, P, OH, OW;
    int ckk, rows;
};

constexpr int kOcPad = 32;  // gy staging pitch: 4 oc per thread x 8 thread rows

// KT: k values per thread (the block covers 32 * KT columns of col); PIX pixels staged per iteration.
template <int KT, int PIX>
__global__ void __launch_bounds__(256) conv_dw_direct_kernel(const float *__restrict__ x, const float *__restrict__ gy,
                                                             float *__restrict__ slices, const DwGeom g, const int layout)
{
    constexpr int KP  = 32 * KT;
    constexpr int KPP = KP + 1;      // odd pitches: the staging threads write down a column without bank conflicts
    constexpr int OCP = kOcPad + 1;
    extern __shared__ float smem[];
    float *col_s = smem;                       // [PIX][KPP]
    float *gy_s  = col_s + PIX * KPP;          // [PIX][OCP]
    int2 *ktab   = reinterpret_cast<int2 *>(smem + ((PIX * (KPP + OCP) + 1) & ~1));  // [KP] {offset, kh << 16 | kw}; y = -1 past ckk
    const int tid = threadIdx.x, tx = tid & 31, ty = tid >> 5;
    for (int k = tid; k < KP; k += 256)
    {
        int2 e = make_int2(0, -1);
        if (k < g.ckk)
        {
            const int khw = g.KH * g.KW;
            const int c = k / khw, rm = k - c * khw, kh = rm / g.KW, kw = rm - kh * g.KW;
            e = make_int2((c * g.H + kh) * g.W + kw, (kh << 16) | kw);
        }
        ktab[k] = e;
    }
    float acc[4][KT];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < KT; ++j)
            acc[i][j] = 0.f;
    const int ohw = g.OH * g.OW;
    __syncthreads();
    for (int r0 = blockIdx.x * PIX; r0 < g.rows; r0 += gridDim.x * PIX)
    {
        // ---- stage: thread (p = tid % PIX, lane group q = tid / PIX) gathers columns q, q + 256/PIX, ... of pixel p
        {
            constexpr int GROUPS = 256 / PIX;
            const int p = tid % PIX, q = tid / PIX;
            const int r = r0 + p;
            const bool ok = r < g.rows;
            int n = 0, oh = 0, ow = 0;
            if (ok)
            {
                ow          = r % g.OW;
                const int t = r / g.OW;
                oh          = t % g.OH;
                n           = t / g.OH;
            }
            const int h0 = oh * g.S - g.P, w0 = ow * g.S - g.P;
            const int pix_off = (n * g.C * g.H + h0) * g.W + w0;
            for (int k = q; k < KP; k += GROUPS)
            {
                const int2 e  = ktab[k];
                const int hh  = h0 + (e.y >> 16), ww = w0 + (e.y & 0xffff);
                const bool in = ok && e.y >= 0 && hh >= 0 && hh < g.H && ww >= 0 && ww < g.W;
                col_s[p * KPP + k] = in ? __ldg(x + pix_off + e.x) : 0.f;
            }
            for (int oc = q; oc < kOcPad; oc += GROUPS)
            {
                float v = 0.f;
                if (ok && oc < g.OC)
                    v = layout == 0 ? __ldg(gy + (static_cast<int64_t>(n) * g.OC + oc) * ohw + (r - n * ohw))
                                    : __ldg(gy + static_cast<int64_t>(r) * g.OC + oc);
                gy_s[p * OCP + oc] = v;
            }
        }
        __syncthreads();
        // ---- accumulate: thread (ty, tx) owns oc = ty + 8 i and k = tx + 32 j
#pragma unroll 4
        for (int p = 0; p < PIX; ++p)
        {
            float gv[4], cv[KT];
#pragma unroll
            for (int i = 0; i < 4; ++i)
                gv[i] = gy_s[p * OCP + ty + 8 * i];
#pragma unroll
            for (int j = 0; j < KT; ++j)
                cv[j] = col_s[p * KPP + tx + 32 * j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < KT; ++j)
                    acc[i][j] = fmaf(gv[i], cv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < KT; ++j)
        {
            const int oc = ty + 8 * i, k = tx + 32 * j;
            if (oc < g.OC && k < g.ckk)
                slices[(static_cast<int64_t>(blockIdx.x) * g.OC + oc) * g.ckk + k] = acc[i][j];
        }
}

template <int KT, int PIX>
int launch_dw(const float *x, const float *gy, float *gw, const DwGeom &g, int layout, cudaStream_t stream)
{
    constexpr int KP   = 32 * KT;
    const size_t smem  = sizeof(float) * (PIX * (KP + 1 + kOcPad + 1) + 2) + sizeof(int2) * KP;
    const int chunks   = (g.rows + PIX - 1) / PIX;
    const int blocks   = chunks < 148 * 4 ? chunks : 148 * 4;
    const int64_t out  = static_cast<int64_t>(g.OC) * g.ckk;
    float *slices      = colsum_partial_scratch(blocks, out);
    if (!slices)
        return kCudaError;
    conv_dw_direct_kernel<KT, PIX><<<blocks, 256, smem, stream>>>(x, gy, slices, g, layout);
    ++g_launch_count;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
    {
        set_last_error("conv_dw_direct_kernel<%d,%d> launch failed: %s", KT, PIX, cudaGetErrorString(e));
        return kCudaError;
    }
    return colsum_finish_launch(slices, blocks, out, (int)out, gw, stream);  // gw += sum of the slices (gw was zeroed)
}
}  // namespace

extern int g_conv_mode;

bool conv_dw_direct_eligible(int64_t N, int64_t C, int64_t H, int64_t W, int64_t OC, int KH, int KW, int OH, int OW)
{
    return g_conv_mode != 1 && g_conv_mode != 2 && OC <= 32 && C * KH * KW <= 256 && N * OH * OW < (int64_t(1) << 31) - 256 &&
           N * C * H * W < (int64_t(1) << 31) - (int64_t(1) << 20);
}

int conv_dw_direct_launch(const float *x, const float *gy, float *gw, int64_t N, int64_t C, int64_t H, int64_t W, int64_t OC,
                          int KH, int KW, int S, int P, int OH, int OW, int layout, cudaStream_t stream)
{
    DwGeom g;
    g.N = (int)N, g.C = (int)C, g.H = (int)H, g.W = (int)W, g.OC = (int)OC, g.KH = KH, g.KW = KW, g.S = S, g.P = P;
    g.OH = OH, g.OW = OW;
    g.ckk  = (int)(C * KH * KW);
    g.rows = (int)(N * OH * OW);
    ODL_CUDA_TRY(cudaMemsetAsync(gw, 0, sizeof(float) * OC * g.ckk, stream));
    if (g.ckk <= 32)
        return launch_dw<1, 64>(x, gy, gw, g, layout, stream);
    if (g.ckk <= 64)
        return launch_dw<2, 64>(x, gy, gw, g, layout, stream);
    if (g.ckk <= 128)
        return launch_dw<4, 64>(x, gy, gw, g, layout, stream);
    return launch_dw<8, 32>(x, gy, gw, g, layout, stream);
}

}  // namespace odl
