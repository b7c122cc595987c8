// Weight gradient of a small conv2d (OC <= 32, C*KH*KW <= 256) from image tiles in shared memory:
//
//   gw[oc, (c,kh,kw)] = sum over output pixels (n,oh,ow) of gy_rows[(n,oh,ow), oc] * x[n, c, oh*S+kh-P, ow*S+kw-P]
//
// (the reference's conv2d_backward for W, src/mat/origin/cpu/conv/conv2d.cpp:534-600: im2col, then gy_rows^T . col).  The
// gather kernel of conv_dw_direct.cu stages the column matrix of a block of pixels -- C*KH*KW values per pixel, each
// fetched through an offset table, with a bounds test per element on the border.  Overlapping windows make that matrix
// many times larger than the pixels it is made of (9x for a 6 x 6 kernel at stride 2), so here a block stages the IMAGE
// instead: the (TH-1)*S+KH by (TW-1)*S+KW window of x under a TH x TW tile of output pixels, every channel, zero where
// the window leaves the image (that is the padding), plus the tile's rows of gy -- plain asynchronous copies, two buffers,
// the next tile in flight while the current one is used.  A thread keeps an 8 (oc) x KPT (k) register tile as in the
// gather kernel and reads its column values straight from the image tile: pixel base + the offset of its k (KPT offsets in
// registers).  No table, no border path, 5-10x fewer staged elements.  Blocks walk the tiles grid-stride and park their
// partial gw (and gb) in their own slice; a second pass adds the slices in a fixed order: same bits every run.
//
// gy_layout 0: gy_rows is the permuted NCHW gradient (the true gradient); 1: the NCHW buffer reinterpreted as
// [N*OH*OW, OC] as the reference does.  Plain fp32 FMAs; summation order differs from the reference's single accumulator
// (tolerance 1e-5, as for the other weight-gradient paths).
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
constexpr int kPix = 128;  // output pixels per tile: 4 rows of 32 or 8 rows of 16, whichever wastes fewer at the edges

struct TileGeom
{
    int N, C, H, W, OC, KH, KW, S, P, OH, OW;
    int ckk;
    int tw_shift;           // tile width = 1 << tw_shift (5 or 4)
    int xh, xw, xwp;        // image window of a tile: rows, columns, row pitch
    int cstride;            // floats from one channel of the window to the next (pitch and stride are chosen so that the
                            // column reads of a warp fall into distinct banks, see choose_pitch)
    int tiles_h, tiles_w;   // tiles per image
    int tiles;              // N * tiles_h * tiles_w
    int pitch;              // floats per block in the slice buffer: OC * ckk of gw, then OC of gb
    int buf_floats;         // floats of one staging buffer (image window + gy rows)
};

__device__ __forceinline__ void cp_async_f32(float *dst_smem, const float *src, bool valid)
{
    const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(dst_smem));
    const int bytes  = valid ? 4 : 0;  // 0 source bytes: the destination is filled with zeros, nothing is read
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}

__device__ __forceinline__ void cp_async_commit()
{
    asm volatile("cp.async.commit_group;" ::: "memory");
}

template <int N>
__device__ __forceinline__ void cp_async_wait()
{
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <int OCP, int KP, int KPT>
__global__ void __launch_bounds__(256, 2) conv_dw_tile_kernel(const float *__restrict__ x, const float *__restrict__ gy,
                                                              float *__restrict__ slices, const TileGeom g, const int layout,
                                                              const int with_gb)
{
    constexpr int TG   = (OCP / 8) * (KP / KPT);  // threads of a group: together they cover the gw tile
    constexpr int G    = 256 / TG;                // groups: each takes every G-th pixel of the tile
    constexpr int OCPP = OCP + 4;
    static_assert(KP % KPT == 0 && TG <= 256 && 256 % TG == 0 && kPix % G == 0, "tile / block shape");
    extern __shared__ float4 smem4[];
    float *smem   = reinterpret_cast<float *>(smem4);
    const int tid = threadIdx.x;
    const int grp = tid / TG, lt = tid % TG;
    const int ocg = lt / (KP / KPT), kg = lt % (KP / KPT);
    const int x_floats = (g.C * g.cstride + 3) & ~3;  // the gy rows behind the image window start 16-byte aligned
    const int tw_mask  = (1 << g.tw_shift) - 1;
    // offsets of this thread's k columns inside the image window (0 for the padded columns: they are never written out)
    int koff[KPT];
#pragma unroll
    for (int j = 0; j < KPT; ++j)
    {
        const int k = KPT * kg + j;
        koff[j]     = 0;
        if (k < g.ckk)
        {
            const int khw = g.KH * g.KW;
            const int c = k / khw, rm = k - c * khw, kh = rm / g.KW, kw = rm - kh * g.KW;
            koff[j] = c * g.cstride + kh * g.xwp + kw;
        }
    }
    float acc[8][KPT];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < KPT; ++j)
            acc[i][j] = 0.f;
    const int b_oc = tid % OCP, b_part = tid / OCP;  // bias gradient on the side: thread (oc, part) adds every (256/OCP)-th pixel
    float gb_acc   = 0.f;
    const int ohw  = g.OH * g.OW;

    auto stage = [&](int tile, float *buf) {
        const int tw_i = tile % g.tiles_w;
        const int t2   = tile / g.tiles_w;
        const int th_i = t2 % g.tiles_h;
        const int n    = t2 / g.tiles_h;
        const int oh0 = th_i * (kPix >> g.tw_shift), ow0 = tw_i << g.tw_shift;
        const int h0 = oh0 * g.S - g.P, w0 = ow0 * g.S - g.P;
        // image window: rows (c, r) of xw floats; consecutive threads take consecutive columns
        const float *xn = x + static_cast<int64_t>(n) * g.C * g.H * g.W;
        const int rows  = g.C * g.xh;
        int col = tid % g.xw, row = tid / g.xw;
        const int dcol = 256 % g.xw, drow = 256 / g.xw;
        while (row < rows)
        {
            const int c = row / g.xh, r = row - c * g.xh;
            const int hh = h0 + r, ww = w0 + col;
            const bool in = hh >= 0 && hh < g.H && ww >= 0 && ww < g.W;
            cp_async_f32(buf + c * g.cstride + r * g.xwp + col, in ? xn + (static_cast<int64_t>(c) * g.H + hh) * g.W + ww : x, in);
            col += dcol, row += drow;
            if (col >= g.xw)
                col -= g.xw, ++row;
        }
        // gy rows of the tile: [pixel][oc]
        float *gs = buf + x_floats;
        if (layout == 0)
        {
            for (int e = tid; e < OCP * kPix; e += 256)
            {
                const int oc = e / kPix, p = e - oc * kPix;
                const int oh = oh0 + (p >> g.tw_shift), ow = ow0 + (p & tw_mask);
                const bool in = oc < g.OC && oh < g.OH && ow < g.OW;
                cp_async_f32(gs + p * OCPP + oc, in ? gy + (static_cast<int64_t>(n) * g.OC + oc) * ohw + oh * g.OW + ow : gy, in);
            }
        }
        else
        {
            for (int e = tid; e < OCP * kPix; e += 256)
            {
                const int p = e / OCP, oc = e - p * OCP;
                const int oh = oh0 + (p >> g.tw_shift), ow = ow0 + (p & tw_mask);
                const bool in = oc < g.OC && oh < g.OH && ow < g.OW;
                cp_async_f32(gs + p * OCPP + oc,
                             in ? gy + (static_cast<int64_t>(n) * ohw + oh * g.OW + ow) * g.OC + oc : gy, in);
            }
        }
        cp_async_commit();
    };

    int tile = blockIdx.x;
    int cur  = 0;
    if (tile < g.tiles)
        stage(tile, smem);
    for (; tile < g.tiles; tile += gridDim.x, cur ^= 1)
    {
        const int next = tile + gridDim.x;
        if (next < g.tiles)
        {
            stage(next, smem + (cur ^ 1) * g.buf_floats);
            cp_async_wait<1>();
        }
        else
            cp_async_wait<0>();
        __syncthreads();  // the current buffer is complete for every thread
        const float *xs = smem + cur * g.buf_floats;
        const float *gs = xs + x_floats;
#pragma unroll 2
        for (int p = grp; p < kPix; p += G)
        {
            const float4 g0   = *reinterpret_cast<const float4 *>(gs + p * OCPP + 8 * ocg);
            const float4 g1   = *reinterpret_cast<const float4 *>(gs + p * OCPP + 8 * ocg + 4);
            const float gv[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
            const float *xp   = xs + (p >> g.tw_shift) * g.S * g.xwp + (p & tw_mask) * g.S;
            float cv[KPT];
#pragma unroll
            for (int j = 0; j < KPT; ++j)
                cv[j] = xp[koff[j]];
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < KPT; ++j)
                    acc[i][j] = fmaf(gv[i], cv[j], acc[i][j]);
        }
        if (with_gb)
#pragma unroll
            for (int p = b_part; p < kPix; p += 256 / OCP)
                gb_acc += gs[p * OCPP + b_oc];  // pixels past the edge of the output were staged as zeros
        __syncthreads();  // everyone is done with the current buffer before the next stage overwrites it
    }
    // ---- the groups add their tiles in group order (a fixed order) into a tile in shared memory
    float *red = smem;  // [OCP][KP]: the staging buffers are dead; the launcher makes sure it fits
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
        __syncthreads();
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

size_t tile_smem_bytes(const TileGeom &g, int OCP, int KP)
{
    const size_t staging = 2 * static_cast<size_t>(g.buf_floats);
    const size_t red     = static_cast<size_t>(OCP) * KP;
    return sizeof(float) * (staging > red ? staging : red);
}

template <int OCP, int KP, int KPT>
int launch_tile(const float *x, const float *gy, float *gw, float *gb, const TileGeom &g, int layout, cudaStream_t stream)
{
    const size_t smem = tile_smem_bytes(g, OCP, KP);
    static size_t attr_smem = 0;  // the largest dynamic shared-memory size the kernel has been allowed so far
    if (smem > 48 * 1024 && smem > attr_smem)
    {
        ODL_CUDA_TRY(cudaFuncSetAttribute(conv_dw_tile_kernel<OCP, KP, KPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_smem = smem;
    }
    int per_sm = 0, dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, conv_dw_tile_kernel<OCP, KP, KPT>, 256, smem) != cudaSuccess || per_sm < 1)
        per_sm = 1;
    const int resident = sms * per_sm;  // one resident wave of blocks walking the tiles grid-stride
    const int blocks   = g.tiles < resident ? g.tiles : resident;
    const int64_t out  = static_cast<int64_t>(g.OC) * g.ckk;
    float *slices      = colsum_partial_scratch(blocks, g.pitch);
    if (!slices)
        return kCudaError;
    conv_dw_tile_kernel<OCP, KP, KPT><<<blocks, 256, smem, stream>>>(x, gy, slices, g, layout, gb != nullptr);
    ++g_launch_count;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
    {
        set_last_error("conv_dw_tile_kernel<%d,%d,%d> launch failed: %s", OCP, KP, KPT, cudaGetErrorString(e));
        return kCudaError;
    }
    // gw (and gb, which sits behind it in every slice) = the slices added in slice order
    return colsum_finish2_launch(slices, blocks, g.pitch, (int)out, gw, g.OC, gb, stream);
}

// Wavefronts of shared memory the column reads of one warp need (the first pixel step; one wavefront serves the lanes whose
// addresses fall into distinct banks or coincide), summed over a thread's KPT reads.
int read_wavefronts(const TileGeom &g, int ocp, int kp, int kpt)
{
    const int kgs = kp / kpt, tg = (ocp / 8) * kgs;
    int total     = 0;
    for (int j = 0; j < kpt; ++j)
    {
        int addr[32];
        for (int lane = 0; lane < 32; ++lane)
        {
            const int grp = lane / tg, lt = lane % tg, kg = lt % kgs;
            const int k = kpt * kg + j, p = grp;  // warp 0, first step: group g works on pixel g
            int off     = 0;
            if (k < g.ckk)
            {
                const int khw = g.KH * g.KW;
                const int c = k / khw, rm = k - c * khw, kh = rm / g.KW, kw = rm - kh * g.KW;
                off = c * g.cstride + kh * g.xwp + kw;
            }
            addr[lane] = off + (p >> g.tw_shift) * g.S * g.xwp + (p & ((1 << g.tw_shift) - 1)) * g.S;
        }
        int worst = 1;
        for (int bank = 0; bank < 32; ++bank)
        {
            int distinct = 0;
            for (int a = 0; a < 32; ++a)
            {
                if ((addr[a] & 31) != bank)
                    continue;
                bool seen = false;
                for (int b = 0; b < a; ++b)
                    seen = seen || addr[b] == addr[a];
                distinct += !seen;
            }
            worst = distinct > worst ? distinct : worst;
        }
        total += worst;
    }
    return total;
}

// Row pitch and channel stride of the image window with the fewest bank conflicts for the k offsets of a warp.
void choose_pitch(TileGeom *g, int ocp, int kp, int kpt)
{
    int best = 1 << 30, best_xwp = g->xw, best_pad = 0;
    for (int xwp = g->xw; xwp < g->xw + 8 && best > kpt; ++xwp)
        for (int pad = 0; pad < 32 && best > kpt; ++pad)
        {
            g->xwp = xwp, g->cstride = g->xh * xwp + pad;
            const int w = read_wavefronts(*g, ocp, kp, kpt);
            if (w < best)
                best = w, best_xwp = xwp, best_pad = pad;
        }
    g->xwp = best_xwp, g->cstride = g->xh * best_xwp + best_pad;
}

void tile_shape(int ckk, int oc, int *ocp, int *kp, int *kpt)
{
    *ocp = oc <= 16 ? 16 : 32;
    *kpt = ckk > 128 && ckk <= 144 ? 9 : 8;
    *kp  = ckk <= 32 ? 32 : ckk <= 64 ? 64 : ckk <= 128 ? 128 : ckk <= 144 ? 144 : 256;
}

bool make_geom(int64_t N, int64_t C, int64_t H, int64_t W, int64_t OC, int KH, int KW, int S, int P, int OH, int OW, TileGeom *out)
{
    TileGeom g;
    g.N = (int)N, g.C = (int)C, g.H = (int)H, g.W = (int)W, g.OC = (int)OC, g.KH = KH, g.KW = KW, g.S = S, g.P = P;
    g.OH = OH, g.OW = OW;
    g.ckk = (int)(C * KH * KW);
    // the last geometry is kept: the pitch search costs tens of microseconds of host time
    static thread_local TileGeom cached;
    static thread_local bool have = false;
    if (have && cached.N == g.N && cached.C == g.C && cached.H == g.H && cached.W == g.W && cached.OC == g.OC && cached.KH == KH &&
        cached.KW == KW && cached.S == S && cached.P == P)
    {
        *out = cached;
        return true;
    }
    // 4 x 32 or 8 x 16 pixels: the shape that covers the output with fewer tiles
    const int64_t t32 = static_cast<int64_t>((OH + 3) / 4) * ((OW + 31) / 32), t16 = static_cast<int64_t>((OH + 7) / 8) * ((OW + 15) / 16);
    g.tw_shift        = t16 < t32 ? 4 : 5;
    const int tw = 1 << g.tw_shift, th = kPix >> g.tw_shift;
    const int64_t xh = static_cast<int64_t>(th - 1) * S + KH, xw = static_cast<int64_t>(tw - 1) * S + KW;
    // both buffers of two resident blocks must fit: 48 KB of image window per buffer at most
    if (C * (xh * (xw + 8) + 32) * 4 > 48 * 1024 || xw > 256)
        return false;
    g.xh = (int)xh, g.xw = (int)xw;
    int ocp_, kp_, kpt_;
    tile_shape(g.ckk, g.OC, &ocp_, &kp_, &kpt_);
    choose_pitch(&g, ocp_, kp_, kpt_);
    const int64_t x_floats = static_cast<int64_t>(C) * g.cstride;
    g.tiles_h = (OH + th - 1) / th, g.tiles_w = (OW + tw - 1) / tw;
    const int64_t tiles = N * g.tiles_h * g.tiles_w;
    if (tiles >= (int64_t(1) << 30))
        return false;
    g.tiles = (int)tiles;
    g.pitch = (int)(OC * g.ckk + OC);
    const int ocp = OC <= 16 ? 16 : 32;
    // a multiple of 4 floats so that the 128-bit reads of the gy rows stay aligned in the second buffer
    g.buf_floats = (int)((x_floats + 3) / 4 * 4) + kPix * (ocp + 4);
    *out = g;
    cached = g, have = true;
    return true;
}
}  // namespace

// Staging the image pays where the windows of neighbouring pixels overlap a lot: measured on the first three layers of the
// reference's CNN (batch 16) against the gather kernel, 0.105 / 0.075 / 0.046 ms against 0.132 / 0.073 / 0.033 ms -- their
// column matrices are 5.6 / 2.1 / 1.0 times the image windows they are made of.  Taken from a factor of 3 up; conv mode 6
// (test hook) keeps the gather kernel, mode 7 takes this one wherever the window fits.
bool conv_dw_tile_eligible(int64_t N, int64_t C, int64_t H, int64_t W, int64_t OC, int KH, int KW, int S, int P, int OH, int OW)
{
    TileGeom g;
    if (g_conv_mode == 6 || !conv_dw_direct_eligible(N, C, H, W, OC, KH, KW, OH, OW) ||
        !make_geom(N, C, H, W, OC, KH, KW, S, P, OH, OW, &g))
        return false;
    return g_conv_mode == 7 || static_cast<int64_t>(g.ckk) * kPix >= 3 * static_cast<int64_t>(g.C) * g.xh * g.xw;
}

// gb (optional; layout 0 only): the bias gradient, summed from the rows of gy the kernel stages anyway.
int conv_dw_tile_launch(const float *x, const float *gy, float *gw, float *gb, int64_t N, int64_t C, int64_t H, int64_t W,
                        int64_t OC, int KH, int KW, int S, int P, int OH, int OW, int layout, cudaStream_t stream)
{
    TileGeom g;
    if (!make_geom(N, C, H, W, OC, KH, KW, S, P, OH, OW, &g))
    {
        set_last_error("conv_dw_tile: the image window of a tile does not fit shared memory");
        return kTooLarge;
    }
    if (gb && layout != 0)
    {
        set_last_error("conv_dw_tile: the bias gradient rides along only in the true gradient layout");
        return kInvalidArgument;
    }
    if (OC <= 16)
    {
        if (g.ckk <= 32)
            return launch_tile<16, 32, 8>(x, gy, gw, gb, g, layout, stream);
        if (g.ckk <= 64)
            return launch_tile<16, 64, 8>(x, gy, gw, gb, g, layout, stream);
        if (g.ckk <= 128)
            return launch_tile<16, 128, 8>(x, gy, gw, gb, g, layout, stream);
        if (g.ckk <= 144)
            return launch_tile<16, 144, 9>(x, gy, gw, gb, g, layout, stream);
        return launch_tile<16, 256, 8>(x, gy, gw, gb, g, layout, stream);
    }
    if (g.ckk <= 32)
        return launch_tile<32, 32, 8>(x, gy, gw, gb, g, layout, stream);
    if (g.ckk <= 64)
        return launch_tile<32, 64, 8>(x, gy, gw, gb, g, layout, stream);
    if (g.ckk <= 128)
        return launch_tile<32, 128, 8>(x, gy, gw, gb, g, layout, stream);
    if (g.ckk <= 144)
        return launch_tile<32, 144, 9>(x, gy, gw, gb, g, layout, stream);
    return launch_tile<32, 256, 8>(x, gy, gw, gb, g, layout, stream);
}

}  // namespace odl
