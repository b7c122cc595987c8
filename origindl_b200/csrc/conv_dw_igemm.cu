// Implicit-GEMM conv2d weight gradient for sm_100a:  gw[OC, C*KH*KW] = sum over output pixels m of
// gy[m, oc] * col[m, k]  with NO column matrix in HBM (the explicit path writes col and its 3xTF32 low part, 2 x 59 MB
// for a 64 -> 64 3x3 layer on 40 x 40 x 16 images, reads them back in a split-K GEMM and needs gy permuted to rows).
//
// The GEMM is computed transposed, D[k, oc] = colT[k, pixels] . gyT[pixels, oc], so that both operands have the
// reduction (pixels) as their contiguous K dimension:
//   A (128 k-rows x 32 pixels per K-block): gathered from x by the eight worker warps straight into the
//     128-byte-swizzled K-major layout tcgen05.mma reads (row r at byte 128 r, 16-byte chunk j at j ^ (r & 7)), with
//     its 3xTF32 low part.  Lanes walk consecutive pixels (coalesced loads along a row of x), a warp owns 16 of the
//     128 k-rows, so every shared-memory store instruction fills one 128-byte row without bank conflicts.
//   B (BN output channels x 32 pixels): gy is NCHW, i.e. for one image already a K-major [OC][OH*OW] matrix; tiles of
//     it and of its low part arrive by TMA from a 2D map over [N*OC][OH*OW] (pixels past the image end read as zeros;
//     rows past OC belong to the next image and only ever reach accumulator columns that are not stored).
// A K-block is 32 consecutive pixels of ONE image.  The K-blocks (N * ceil(OH*OW / 32)) are divided among gridDim.y
// splits of at most 16 blocks each (the accumulator stays in TMEM for the CTA's whole range: truncating accumulation
// costs about 7.5e-9 per accumulated element relative to the largest result); split z stores its partial gw into slice z
// of a scratch buffer and a second pass adds the slices in order, so the result has the same bits on every run.
// warp 0 lane 0: TMA producer; warp 1 lane 0: MMA issuer; warps 2..9: gather, then epilogue.  Every wait is bounded.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstring>

#include "gemm_epilogue.cuh"
#include "gemm_tc.cuh"
#include "host_util.h"
#include "internal.h"
#include "ptx_sm100.cuh"
#include "tmap.h"

namespace odl
{
namespace
{
constexpr int kBM       = 128;  // k-rows (c, kh, kw) per CTA
constexpr int kBK       = 32;   // pixels per K-block
constexpr int kUmmaK    = 8;
constexpr int kWorkers  = 8;
constexpr int kThreads  = 64 + 32 * kWorkers;
constexpr int kStages   = 2;
constexpr int kAuxBytes = 256;
constexpr int kMaxKb    = 16;   // K-blocks one CTA accumulates in TMEM (512 pixels: 3.8e-6 of truncation error)

struct DwGeom
{
    int N, C, H, W, KH, KW, S, P, OH, OW;
    int ckk;            // C*KH*KW = rows of D
    int ohw;            // OH*OW
    int chunks;         // ceil(ohw / 32): K-blocks per image
    int total_kb;       // N * chunks
    int kb_per_split;
    int64_t slice;      // floats per split slice of the scratch output (OC * ckk)
};

template <int BN>
struct DwCfg
{
    static constexpr int a_bytes     = kBM * kBK * 4;
    static constexpr int b_bytes     = BN * kBK * 4;
    static constexpr int stage_bytes = 2 * (a_bytes + b_bytes);  // A, A_small, B, B_small
    static constexpr int smem_bytes  = 1024 + kStages * stage_bytes + kAuxBytes + kBM * 8;
    static constexpr int tmem_cols   = BN < 32 ? 32 : BN;
    static constexpr int warp_cols   = BN / 2;
};

template <int BN>
__global__ void __launch_bounds__(kThreads, 2)
conv_dw_igemm_kernel(const __grid_constant__ TmapPack tm, const float *__restrict__ x, const DwGeom g, GemmParams p,
                     const int terms)
{
    using Cfg = DwCfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *base       = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *tiles      = base;
    float *stg_all      = reinterpret_cast<float *>(base);  // transpose slabs of the epilogue, after the ring is dead
    uint64_t *b_full    = reinterpret_cast<uint64_t *>(base + kStages * Cfg::stage_bytes);
    uint64_t *a_full    = b_full + kStages;
    uint64_t *empty_bar = a_full + kStages;
    uint64_t *acc_full  = empty_bar + kStages;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_full + 1);
    volatile int *abort_f = reinterpret_cast<volatile int *>(tmem_slot + 1);
    int *early_out        = const_cast<int *>(abort_f) + 1;
    int2 *ktab            = reinterpret_cast<int2 *>(base + kStages * Cfg::stage_bytes + kAuxBytes);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    if (threadIdx.x == 0)
    {
        *early_out = (p.err != nullptr && *reinterpret_cast<volatile int *>(p.err) != 0) ? 1 : 0;
        *abort_f   = 0;
    }
    __syncthreads();
    if (*early_out)
        return;

    const int tiles_n = (p.N + BN - 1) / BN;
    const int tile_m  = blockIdx.x / tiles_n;
    const int tile_n  = blockIdx.x - tile_m * tiles_n;
    const int m0 = tile_m * kBM, n0 = tile_n * BN;
    const int kb0    = blockIdx.y * g.kb_per_split;
    const int num_kb = min(g.kb_per_split, g.total_kb - kb0);
    p.D += static_cast<size_t>(blockIdx.y) * g.slice;  // this split's slice

    // Per-row table of this CTA's 128 k-rows: x[n, c, h0 + kh, w0 + kw] sits at pix_off + ktab[r].x with
    // ktab[r].x = (c * H + kh) * W + kw; ktab[r].y = kh << 16 | kw for the bounds checks; y = -1 past C*KH*KW.
    for (int r = threadIdx.x; r < kBM; r += kThreads)
    {
        int2 e      = make_int2(0, -1);
        const int k = m0 + r;
        if (k < g.ckk)
        {
            const int khw = g.KH * g.KW;
            const int c = k / khw, rm = k - c * khw, kh = rm / g.KW, kw = rm - kh * g.KW;
            e = make_int2((c * g.H + kh) * g.W + kw, (kh << 16) | kw);
        }
        ktab[r] = e;
    }
    if (warp == 0 && lane == 0)
    {
        ptx::prefetch_tmap(&tm.b);
        if (terms == 3)
            ptx::prefetch_tmap(&tm.b_small);
        for (int s = 0; s < kStages; ++s)
        {
            ptx::mbar_init(&b_full[s], 1);
            ptx::mbar_init(&a_full[s], kWorkers);
            ptx::mbar_init(&empty_bar[s], 1);
        }
        ptx::mbar_init(acc_full, 1);
        ptx::fence_mbar_init();
    }
    if (warp == 1)
    {
        ptx::tmem_alloc(tmem_slot, Cfg::tmem_cols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0)
    {
        // ================================================================= TMA producer: gy tiles
        if (lane == 0)
        {
            int issued = 0;
            for (int kb = 0; kb < num_kb; ++kb)
            {
                const int s = kb % kStages;
                if (!ptx::mbar_wait_quiet(&empty_bar[s], ((kb / kStages) & 1) ^ 1, abort_f))
                    break;
                const int kbg = kb0 + kb, img = kbg / g.chunks, chunk = kbg - img * g.chunks;
                uint8_t *sb   = tiles + s * Cfg::stage_bytes + 2 * Cfg::a_bytes;
                ptx::mbar_arrive_expect_tx(&b_full[s], Cfg::b_bytes * (terms == 3 ? 2 : 1));
                ptx::tma_load_2d(sb, &tm.b, &b_full[s], chunk * kBK, img * p.N + n0);
                if (terms == 3)
                    ptx::tma_load_2d(sb + Cfg::b_bytes, &tm.b_small, &b_full[s], chunk * kBK, img * p.N + n0);
                ++issued;
            }
            if (*abort_f)
            {
                const int first = issued > kStages ? issued - kStages : 0;
                for (int kb = first; kb < issued; ++kb)
                    ptx::mbar_wait_quiet(&b_full[kb % kStages], (kb / kStages) & 1, nullptr);
            }
        }
    }
    else if (warp == 1)
    {
        // ================================================================= MMA issuer
        if (lane == 0)
        {
            const uint32_t idesc = ptx::make_idesc_tf32(kBM, BN < 16 ? 16 : BN, false, false);
            bool ok              = true;
            for (int kb = 0; kb < num_kb && ok; ++kb)
            {
                const int s       = kb % kStages;
                const uint32_t ph = (kb / kStages) & 1;
                if (!ptx::mbar_wait_quiet(&a_full[s], ph, abort_f) || !ptx::mbar_wait_quiet(&b_full[s], ph, abort_f))
                {
                    ok = false;
                    break;
                }
                ptx::tc_fence_after_sync();
                const uint32_t sa  = ptx::smem_u32(tiles + s * Cfg::stage_bytes);
                const uint32_t sas = sa + Cfg::a_bytes;
                const uint32_t sb  = sa + 2 * Cfg::a_bytes;
                const uint32_t sbs = sb + Cfg::b_bytes;
#pragma unroll
                for (int kk = 0; kk < kBK / kUmmaK; ++kk)
                {
                    const uint32_t acc_on = (kb > 0 || kk > 0) ? 1u : 0u;
                    const uint64_t da = ptx::make_smem_desc(sa + kk * 32, 16, 1024, ptx::kLayoutSw128);
                    const uint64_t db = ptx::make_smem_desc(sb + kk * 32, 16, 1024, ptx::kLayoutSw128);
                    if (terms == 3)
                    {
                        const uint64_t das = ptx::make_smem_desc(sas + kk * 32, 16, 1024, ptx::kLayoutSw128);
                        const uint64_t dbs = ptx::make_smem_desc(sbs + kk * 32, 16, 1024, ptx::kLayoutSw128);
                        ptx::mma_tf32_ss(tmem_base, das, db, idesc, acc_on);
                        ptx::mma_tf32_ss(tmem_base, da, dbs, idesc, 1);
                        ptx::mma_tf32_ss(tmem_base, da, db, idesc, 1);
                    }
                    else
                    {
                        ptx::mma_tf32_ss(tmem_base, da, db, idesc, acc_on);
                    }
                }
                ptx::mma_commit(&empty_bar[s]);
            }
            if (ok)
                ptx::mma_commit(acc_full);
        }
    }
    else
    {
        // ================================================================= gather (im2col on the fly), then epilogue
        const int e = warp - 2;   // this warp gathers k-rows 16 e .. 16 e + 15 of the tile
        const int q = warp & 3;   // TMEM lane quarter this warp may read
        const int h = e >> 2;     // half of the tile's columns it stores in the epilogue
        bool have   = true;
        // The 16 values of K-block kb are loaded into registers one K-block ahead of the stores.
        auto gather = [&](int kb, float (&v)[16]) {
            const int kbg = kb0 + kb, img = kbg / g.chunks, chunk = kbg - img * g.chunks;
            const int pix = chunk * kBK + lane;           // this lane's pixel of image img
            const bool pix_ok = pix < g.ohw;
            const int oh = pix / g.OW, ow = pix - oh * g.OW;
            const int h0 = oh * g.S - g.P, w0 = ow * g.S - g.P;
            const int pix_off = (img * g.C * g.H + h0) * g.W + w0;
            const bool interior = pix_ok && h0 >= 0 && h0 + g.KH <= g.H && w0 >= 0 && w0 + g.KW <= g.W;
            const int2 *tab     = ktab + 16 * e;
            if (__all_sync(0xffffffffu, interior))
            {
#pragma unroll
                for (int i = 0; i < 16; ++i)
                {
                    const int2 t = tab[i];
                    v[i]         = t.y >= 0 ? __ldg(x + pix_off + t.x) : 0.f;
                }
            }
            else
            {
#pragma unroll
                for (int i = 0; i < 16; ++i)
                {
                    const int2 t  = tab[i];
                    const int hh  = h0 + (t.y >> 16), ww = w0 + (t.y & 0xffff);
                    const bool in = pix_ok && t.y >= 0 && hh >= 0 && hh < g.H && ww >= 0 && ww < g.W;
                    v[i]          = in ? __ldg(x + pix_off + t.x) : 0.f;
                }
            }
        };
        float v[16], v_next[16];
        if (num_kb > 0)
            gather(0, v_next);
        for (int kb = 0; kb < num_kb; ++kb)
        {
            const int s = kb % kStages;
#pragma unroll
            for (int i = 0; i < 16; ++i)
                v[i] = v_next[i];
            if (kb + 1 < num_kb)
                gather(kb + 1, v_next);
            have = __all_sync(0xffffffffu, ptx::mbar_wait_quiet(&empty_bar[s], ((kb / kStages) & 1) ^ 1, abort_f));
            if (!have)
                break;
            uint8_t *a_big   = tiles + s * Cfg::stage_bytes;
            uint8_t *a_small = a_big + Cfg::a_bytes;
#pragma unroll
            for (int i = 0; i < 16; ++i)
            {
                const int r   = 16 * e + i;  // tile row; this lane's pixel is column `lane` of the K-block
                const int off = r * 128 + (((lane >> 2) ^ (r & 7)) << 4) + ((lane & 3) << 2);
                *reinterpret_cast<float *>(a_big + off) = v[i];
                if (terms == 3)
                    *reinterpret_cast<float *>(a_small + off) = tf32_small(v[i]);
            }
            ptx::fence_proxy_async_smem();  // generic-proxy writes -> visible to the tensor core's reads
            __syncwarp();
            if (lane == 0)
                ptx::mbar_arrive(&a_full[s]);
        }
        if (have)
            have = __all_sync(0xffffffffu, ptx::mbar_wait_quiet(acc_full, 0, abort_f));
        if (have)
        {
            ptx::tc_fence_after_sync();
            const int cw = h * Cfg::warp_cols;
            float acc[Cfg::warp_cols];
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(32 * q) << 16) + cw;
#pragma unroll
            for (int j = 0; j < Cfg::warp_cols / 32; ++j)
            {
                uint32_t rr[32];
                ptx::tmem_ld_32x32(taddr + 32 * j, rr);
                ptx::tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    acc[32 * j + i] = __uint_as_float(rr[i]);
            }
            // "NCHW" store with one image of ckk "pixels": row m = k goes to D[oc * ckk + k] -- gw's own layout
            gemm_epilogue_store<BN, Cfg::warp_cols>(p, acc, stg_all + e * 32 * kStgLd, m0, n0, cw, q, lane);
        }
        ptx::tc_fence_before_sync();
    }

    __syncthreads();
    if (warp == 1)
    {
        __syncwarp();
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, Cfg::tmem_cols);
    }
    if (threadIdx.x == 0 && *abort_f && p.err != nullptr)
        atomicExch(p.err, 1);
}

template <int BN>
int launch_dw(const TmapPack &tm, const float *x, const DwGeom &g, const GemmParams &p, int splits, int terms,
              cudaStream_t stream)
{
    using Cfg = DwCfg<BN>;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    dev &= 63;
    if (!attr_set[dev])
    {
        cudaError_t e = cudaFuncSetAttribute(conv_dw_igemm_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::smem_bytes);
        if (e != cudaSuccess)
        {
            set_last_error("cudaFuncSetAttribute(conv_dw_igemm, smem=%d) failed: %s", Cfg::smem_bytes, cudaGetErrorString(e));
            return kCudaError;
        }
        attr_set[dev] = true;
    }
    const int tiles_m = (g.ckk + kBM - 1) / kBM, tiles_n = (p.N + BN - 1) / BN;
    conv_dw_igemm_kernel<BN><<<dim3(tiles_m * tiles_n, splits), kThreads, Cfg::smem_bytes, stream>>>(tm, x, g, p, terms);
    ++g_launch_count;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
    {
        set_last_error("conv_dw_igemm_kernel<%d> launch failed: %s", BN, cudaGetErrorString(e));
        return kCudaError;
    }
    return kOk;
}
}  // namespace

extern int g_conv_mode;

bool conv_dw_igemm_eligible(int64_t N, int64_t C, int64_t H, int64_t W, int64_t OC, int KH, int KW, int OH, int OW)
{
    const int64_t ohw = static_cast<int64_t>(OH) * OW, ckk = C * KH * KW;
    const int64_t chunks = (ohw + kBK - 1) / kBK;
    // the TMA map over gy needs a 16-byte row pitch; 32-bit element offsets into x; a bounded number of splits
    return g_conv_mode != 1 && (ohw & 3) == 0 && N * C * H * W < (int64_t(1) << 31) - (int64_t(1) << 20) &&
           N * OC < (int64_t(1) << 31) && ckk * OC <= (int64_t(1) << 24) && N * chunks <= 60000 * int64_t(kMaxKb);
}

namespace
{
// K-blocks per split: enough splits that no CTA accumulates more than kMaxKb blocks in TMEM, then as many as fill the
// last wave of CTAs (two per SM) they start.
int plan_kb_per_split(int64_t total_kb, int64_t tiles)
{
    const int64_t slots  = 296;
    const int64_t needed = (total_kb + kMaxKb - 1) / kMaxKb;
    const int64_t waves  = (tiles * needed + slots - 1) / slots;
    int64_t splits       = waves * slots / tiles;
    if (splits < needed)
        splits = needed;
    if (splits > total_kb)
        splits = total_kb;
    if (splits < 1)
        splits = 1;
    return static_cast<int>((total_kb + splits - 1) / splits);
}
}  // namespace

// Number of floats of scratch conv_dw_igemm_launch needs for its split slices.
size_t conv_dw_igemm_scratch(int64_t N, int64_t C, int64_t OC, int KH, int KW, int OH, int OW)
{
    const int64_t ckk = C * KH * KW, chunks = (static_cast<int64_t>(OH) * OW + kBK - 1) / kBK, total_kb = N * chunks;
    const int bn      = OC <= 64 ? 64 : 128;
    const int64_t tiles = ((ckk + kBM - 1) / kBM) * ((OC + bn - 1) / bn);
    const int64_t per    = plan_kb_per_split(total_kb, tiles);
    const int64_t splits = (total_kb + per - 1) / per;
    return static_cast<size_t>(splits) * OC * ckk;
}

// gy: NCHW gradient; gy_small: its 3xTF32 low part (same layout; null in plain TF32); slices: scratch of
// conv_dw_igemm_scratch(...) floats; gw[OC][C*KH*KW] is overwritten.
int conv_dw_igemm_launch(const float *x, const float *gy, const float *gy_small, float *slices, float *gw, int64_t N,
                         int64_t C, int64_t H, int64_t W, int64_t OC, int KH, int KW, int S, int P, int OH, int OW, int terms,
                         cudaStream_t stream)
{
    DwGeom g;
    g.N = (int)N, g.C = (int)C, g.H = (int)H, g.W = (int)W, g.KH = KH, g.KW = KW, g.S = S, g.P = P, g.OH = OH, g.OW = OW;
    g.ckk      = (int)(C * KH * KW);
    g.ohw      = OH * OW;
    g.chunks   = (g.ohw + kBK - 1) / kBK;
    g.total_kb = g.N * g.chunks;
    g.slice    = OC * static_cast<int64_t>(g.ckk);
    const int bn      = OC <= 64 ? 64 : 128;
    const int tiles   = ((g.ckk + kBM - 1) / kBM) * (((int)OC + bn - 1) / bn);
    g.kb_per_split    = plan_kb_per_split(g.total_kb, tiles);
    const int splits = (g.total_kb + g.kb_per_split - 1) / g.kb_per_split;
    GemmParams p;
    std::memset(&p, 0, sizeof(p));
    p.D   = splits > 1 ? slices : gw;
    p.err = device_error_flag();
    p.M = g.ckk, p.N = (int)OC, p.K = g.total_kb * kBK;
    p.ldd   = (int)OC;
    p.flags = kEpiNCHW;
    p.ohw   = g.ckk;  // one "image" of ckk rows: D[oc * ckk + k]
    TmapPack tm;
    std::memset(&tm, 0, sizeof(tm));
    int rc;
    if ((rc = make_tmap(&tm.b, gy, N * OC, g.ohw, g.ohw, kBK, bn, CU_TENSOR_MAP_SWIZZLE_128B)))
        return rc;
    if (terms == 3 && (rc = make_tmap(&tm.b_small, gy_small, N * OC, g.ohw, g.ohw, kBK, bn, CU_TENSOR_MAP_SWIZZLE_128B)))
        return rc;
    rc = bn == 64 ? launch_dw<64>(tm, x, g, p, splits, terms, stream) : launch_dw<128>(tm, x, g, p, splits, terms, stream);
    if (rc || splits == 1)
        return rc;
    return splitk_sum_launch(slices, splits, (int)OC, g.ckk, g.ckk, gw, g.ckk, stream);
}

}  // namespace odl
