// Weight gradient of conv2d without a column matrix in HBM, for small convolutions (OC <= 32, C*KH*KW <= 256):
//
//   gw[oc, k] = sum over output pixels r of gy_rows[r, oc] * col[r, k],   col[r, (c,kh,kw)] = x[n, c, oh*S+kh-P, ow*S+kw-P]
//
// (the reference's conv2d_backward for W, src/mat/origin/cpu/conv/conv2d.cpp:534-600: im2col, then gy_rows^T . col).  The
// explicit path writes col and its 3xTF32 low part to HBM (2 x 177 MB for the first conv layer of the reference's CNN),
// reads them back in a split-K GEMM whose 16 x 108 output uses a fraction of one tensor-core tile, and needs gy
// re-laid out as rows.  Here a block stages PIX pixels of gy and of col in shared memory (col gathered from x through a
// per-block table k -> offset, like the implicit-GEMM forward) and every thread keeps an 8 x 8 register tile of
// (oc, k) sums in plain fp32 FMAs (see the kernel for how the threads share the pixels); blocks walk the pixels
// grid-stride, store their partial gw into their own slice of a scratch buffer, and a second pass adds the slices in a
// fixed order (same bits every run).  The work is N*OH*OW * OC * C*KH*KW FMAs (0.7 G for that layer) on the CUDA cores.
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
    int pitch;  // floats per block in the slice buffer: OC * ckk of gw, then OC of gb
};

// OCP: output channels of the tile (16 or 32, OC padded up); KP: k columns of the tile (32 .. 256, C*KH*KW padded up);
// PIX: pixels staged per iteration; KPT: k columns per thread (8, or 9 for the 144 = 16 x 3 x 3 columns of a 3 x 3 conv over
// 16 channels, which a 256-wide tile would pad by 78 %).  A thread owns an 8 (oc) x KPT (k) register tile, so the (OCP / 8) x (KP / KPT) threads of
// one GROUP cover the whole gw tile; the 256 / that many groups of the block each take every G-th staged pixel, and add
// their tiles in group order at the end.  Per pixel a thread reads 8 gy values and 8 column values (four 128-bit
// shared-memory reads) for 64 multiply-adds: the kernel is bound by FMA issue, not by shared memory.
template <int OCP, int KP, int PIX, int KPT>
__global__ void __launch_bounds__(256, (KP <= 144 ? 2 : 1)) conv_dw_direct_kernel(const float *__restrict__ x, const float *__restrict__ gy,
                                                             float *__restrict__ slices, const DwGeom g, const int layout,
                                                             const int with_gb)
{
    constexpr int TG   = (OCP / 8) * (KP / KPT);  // threads of a group
    static_assert(KP % KPT == 0 && KP % 4 == 0, "k columns per thread / per staging chunk");
    constexpr int G    = 256 / TG;              // groups = pixels in flight per accumulate step
    constexpr int KPP  = KP + 4;                // pitches keep 16-byte alignment; + 4 floats: the 128-bit staging stores
    constexpr int OCPP = OCP + 4;               // of 8 consecutive pixels fall into distinct 16-byte bank groups
    static_assert(TG <= 256 && 256 % TG == 0 && PIX % G == 0 && 256 % PIX == 0, "tile / block shape");
    extern __shared__ float4 smem4[];
    float *col_s = reinterpret_cast<float *>(smem4);                  // [PIX][KPP]
    float *gy_s  = col_s + PIX * KPP;                                 // [PIX][OCPP]
    int2 *ktab   = reinterpret_cast<int2 *>(gy_s + PIX * OCPP);       // [KP] {offset, kh << 16 | kw}; y = -1 past ckk
    const int tid = threadIdx.x;
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
    const int grp = tid / TG, lt = tid % TG;
    const int ocg = lt / (KP / KPT), kg = lt % (KP / KPT);
    float acc[8][KPT];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < KPT; ++j)
            acc[i][j] = 0.f;
    const int ohw = g.OH * g.OW;
    // ---- staging, one iteration ahead through registers: thread (p = tid % PIX, q = tid / PIX) gathers the 4-column chunks
    //      q, q + Q, ... of pixel p (consecutive threads = consecutive pixels: every global load of a tap is coalesced, stride
    //      S).  All loads of the NEXT PIX pixels are issued before the multiply-adds of the current ones, so their latency
    //      hides behind the arithmetic instead of standing between two barriers.
    constexpr int Q   = 256 / PIX;
    constexpr int CH  = (KP / 4) / Q;   // column chunks per thread
    constexpr int GCH = (OCP / 4 + Q - 1) / Q;  // gy chunks per thread
    static_assert((KP / 4) % Q == 0, "column chunks divide evenly over the staging threads");
    const int sp = tid % PIX, sq = tid / PIX;
    float vcol[CH][4], vgy[GCH][4];
    auto gather = [&](int r0) {
        const int r   = r0 + sp;
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
        const bool inside = ok && h0 >= 0 && h0 + g.KH <= g.H && w0 >= 0 && w0 + g.KW <= g.W;
        if (__all_sync(0xffffffffu, inside))
        {
            // every pixel of the warp has its whole window inside the image (all but the border rows and columns): one
            // table read, one add and one load per element.  The padded columns k >= ckk read offset 0 of the window --
            // whatever they accumulate is never written out.
#pragma unroll
            for (int c = 0; c < CH; ++c)
            {
                const int4 *tp = reinterpret_cast<const int4 *>(ktab + 4 * (sq + c * Q));
                const int4 e01 = tp[0], e23 = tp[1];
                vcol[c][0]     = __ldg(x + pix_off + e01.x);
                vcol[c][1]     = __ldg(x + pix_off + e01.z);
                vcol[c][2]     = __ldg(x + pix_off + e23.x);
                vcol[c][3]     = __ldg(x + pix_off + e23.z);
            }
        }
        else
        {
#pragma unroll
            for (int c = 0; c < CH; ++c)
            {
                const int ch = sq + c * Q;
#pragma unroll
                for (int j = 0; j < 4; ++j)
                {
                    const int2 e = ktab[4 * ch + j];
                    bool in      = inside && e.y >= 0;
                    if (!inside && ok && e.y >= 0)
                    {
                        const int hh = h0 + (e.y >> 16), ww = w0 + (e.y & 0xffff);
                        in           = hh >= 0 && hh < g.H && ww >= 0 && ww < g.W;
                    }
                    vcol[c][j] = in ? __ldg(x + pix_off + e.x) : 0.f;
                }
            }
        }
#pragma unroll
        for (int c = 0; c < GCH; ++c)
        {
            const int ch = sq + c * Q;
#pragma unroll
            for (int j = 0; j < 4; ++j)
            {
                const int oc = 4 * ch + j;
                vgy[c][j]    = 0.f;
                if (ok && ch < OCP / 4 && oc < g.OC)
                    vgy[c][j] = layout == 0 ? __ldg(gy + (static_cast<int64_t>(n) * g.OC + oc) * ohw + (r - n * ohw))
                                            : __ldg(gy + static_cast<int64_t>(r) * g.OC + oc);
            }
        }
    };
    __syncthreads();  // ktab is complete
    // bias gradient on the side (with_gb; layout 0 only, where a staged row of gy is one pixel's channels): thread
    // (oc = tid % OCP, part = tid / OCP) adds the pixels part, part + 256 / OCP, ... of every staged block
    const int b_oc = tid % OCP, b_part = tid / OCP;
    float gb_acc   = 0.f;
    const int step = gridDim.x * PIX;
    int r0         = blockIdx.x * PIX;
    if (r0 < g.rows)
        gather(r0);
    for (; r0 < g.rows; r0 += step)
    {
#pragma unroll
        for (int c = 0; c < CH; ++c)
            *reinterpret_cast<float4 *>(col_s + sp * KPP + 4 * (sq + c * Q)) =
                make_float4(vcol[c][0], vcol[c][1], vcol[c][2], vcol[c][3]);
#pragma unroll
        for (int c = 0; c < GCH; ++c)
            if (sq + c * Q < OCP / 4)
                *reinterpret_cast<float4 *>(gy_s + sp * OCPP + 4 * (sq + c * Q)) =
                    make_float4(vgy[c][0], vgy[c][1], vgy[c][2], vgy[c][3]);
        __syncthreads();
        if (r0 + step < g.rows)
            gather(r0 + step);  // in flight during the multiply-adds below
        // ---- accumulate: this group's pixels grp, grp + G, ...
#pragma unroll 2
        for (int p = grp; p < PIX; p += G)
        {
            const float4 g0 = *reinterpret_cast<const float4 *>(gy_s + p * OCPP + 8 * ocg);
            const float4 g1 = *reinterpret_cast<const float4 *>(gy_s + p * OCPP + 8 * ocg + 4);
            const float gv[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
            float cv[KPT];
            if (KPT == 8)
            {
                const float4 c0 = *reinterpret_cast<const float4 *>(col_s + p * KPP + 8 * kg);
                const float4 c1 = *reinterpret_cast<const float4 *>(col_s + p * KPP + 8 * kg + 4);
                cv[0] = c0.x, cv[1] = c0.y, cv[2] = c0.z, cv[3] = c0.w, cv[4] = c1.x, cv[5] = c1.y, cv[6] = c1.z, cv[7] = c1.w;
            }
            else
            {
                // an odd stride: scalar reads, the KP / KPT threads of a row on distinct banks
#pragma unroll
                for (int j = 0; j < KPT; ++j)
                    cv[j] = col_s[p * KPP + KPT * kg + j];
            }
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < KPT; ++j)
                    acc[i][j] = fmaf(gv[i], cv[j], acc[i][j]);
        }
        if (with_gb)
#pragma unroll
            for (int p = b_part; p < PIX; p += 256 / OCP)
                gb_acc += gy_s[p * OCPP + b_oc];  // rows past the last pixel were staged as zeros
        __syncthreads();
    }
    // ---- the groups add their tiles in group order (a fixed order: same bits every run) into a tile in shared memory
    float *red = col_s;  // [OCP][KP]; the staging area is dead (OCP * KP <= PIX * KPP is checked by the launcher's choice of PIX)
    for (int gi = 0; gi < G; ++gi)
    {
        if (grp == gi)
        {
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < KPT; ++j)
                {
                    float *dst = red + (8 * ocg + i) * KP + KPT * kg + j;
                    *dst       = gi == 0 ? acc[i][j] : *dst + acc[i][j];
                }
        }
        __syncthreads();
    }
    for (int o = tid; o < OCP * KP; o += 256)
    {
        const int oc = o / KP, k = o - oc * KP;
        if (oc < g.OC && k < g.ckk)
            slices[static_cast<int64_t>(blockIdx.x) * g.pitch + oc * g.ckk + k] = red[o];
    }
    if (with_gb)
    {
        __syncthreads();  // the gw tile has been read
        red[b_part * OCP + b_oc] = gb_acc;
        __syncthreads();
        if (tid < g.OC)
        {
            float s = 0.f;
            for (int part = 0; part < 256 / OCP; ++part)
                s += red[part * OCP + tid];
            slices[static_cast<int64_t>(blockIdx.x) * g.pitch + g.OC * g.ckk + tid] = s;
        }
    }
}

template <int OCP, int KP, int PIX, int KPT = 8>
int launch_dw(const float *x, const float *gy, float *gw, float *gb, const DwGeom &g, int layout, cudaStream_t stream)
{
    static_assert(OCP * KP <= PIX * (KP + 4), "the reduction tile reuses the column staging area");
    const size_t smem  = sizeof(float) * (PIX * (KP + 4) + PIX * (OCP + 4)) + sizeof(int2) * KP;
    const int chunks   = (g.rows + PIX - 1) / PIX;
    // one resident wave of blocks walking the pixels grid-stride: as many blocks as the GPU holds at once
    static int resident = 0;
    if (resident == 0)
    {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(conv_dw_direct_kernel<OCP, KP, PIX, KPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        int per_sm = 0, dev = 0, sms = 148;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, conv_dw_direct_kernel<OCP, KP, PIX, KPT>, 256, smem) != cudaSuccess ||
            per_sm < 1)
            per_sm = 1;
        resident = sms * per_sm;
    }
    const int blocks   = chunks < resident ? chunks : resident;
    const int64_t out  = static_cast<int64_t>(g.OC) * g.ckk;
    float *slices      = colsum_partial_scratch(blocks, g.pitch);
    if (!slices)
        return kCudaError;
    conv_dw_direct_kernel<OCP, KP, PIX, KPT><<<blocks, 256, smem, stream>>>(x, gy, slices, g, layout, gb != nullptr);
    ++g_launch_count;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
    {
        set_last_error("conv_dw_direct_kernel<%d,%d,%d> launch failed: %s", OCP, KP, PIX, cudaGetErrorString(e));
        return kCudaError;
    }
    // gw (and gb, which sits behind it in every slice) = the slices added in slice order
    return colsum_finish2_launch(slices, blocks, g.pitch, (int)out, gw, g.OC, gb, stream);
}
}  // namespace

extern int g_conv_mode;

bool conv_dw_direct_eligible(int64_t N, int64_t C, int64_t H, int64_t W, int64_t OC, int KH, int KW, int OH, int OW)
{
    return g_conv_mode != 1 && g_conv_mode != 2 && OC <= 32 && C * KH * KW <= 256 && N * OH * OW < (int64_t(1) << 31) - 256 &&
           N * C * H * W < (int64_t(1) << 31) - (int64_t(1) << 20);
}

// gb (optional; layout 0 only): the bias gradient, summed from the rows of gy the kernel stages anyway.
int conv_dw_direct_launch(const float *x, const float *gy, float *gw, float *gb, int64_t N, int64_t C, int64_t H, int64_t W,
                          int64_t OC, int KH, int KW, int S, int P, int OH, int OW, int layout, cudaStream_t stream)
{
    if (gb && layout != 0)
    {
        set_last_error("conv_dw_direct: the bias gradient rides along only in the true gradient layout");
        return kInvalidArgument;
    }
    DwGeom g;
    g.N = (int)N, g.C = (int)C, g.H = (int)H, g.W = (int)W, g.OC = (int)OC, g.KH = KH, g.KW = KW, g.S = S, g.P = P;
    g.OH = OH, g.OW = OW;
    g.ckk  = (int)(C * KH * KW);
    g.rows  = (int)(N * OH * OW);
    g.pitch = (int)(OC * g.ckk + OC);
    if (OC <= 16)
    {
        if (g.ckk <= 32)
            return launch_dw<16, 32, 64>(x, gy, gw, gb, g, layout, stream);
        if (g.ckk <= 64)
            return launch_dw<16, 64, 64>(x, gy, gw, gb, g, layout, stream);
        if (g.ckk <= 128)
            return launch_dw<16, 128, 64>(x, gy, gw, gb, g, layout, stream);
        if (g.ckk <= 144)
            return launch_dw<16, 144, 64, 9>(x, gy, gw, gb, g, layout, stream);
        return launch_dw<16, 256, 64>(x, gy, gw, gb, g, layout, stream);
    }
    if (g.ckk <= 32)
        return launch_dw<32, 32, 64>(x, gy, gw, gb, g, layout, stream);
    if (g.ckk <= 64)
        return launch_dw<32, 64, 64>(x, gy, gw, gb, g, layout, stream);
    if (g.ckk <= 128)
        return launch_dw<32, 128, 64>(x, gy, gw, gb, g, layout, stream);
    if (g.ckk <= 144)
        return launch_dw<32, 144, 64, 9>(x, gy, gw, gb, g, layout, stream);
    return launch_dw<32, 256, 64>(x, gy, gw, gb, g, layout, stream);
}

}  // namespace odl
