// Implicit-GEMM conv2d forward for sm_100a: y[N,OC,OH,OW] = act(scale * conv2d(x[N,C,H,W], w[OC,C,KH,KW]) + b) with the
// tcgen05 tensor core and NO column matrix.
//
// The GEMM is D[pixels, OC] = col[pixels, C*KH*KW] . w[OC, C*KH*KW]^T.  The explicit path (im2col kernel + GEMM) writes
// col and its 3xTF32 low part to HBM and reads them back -- for the first conv layer of the reference's CNN 2 x 177 MB
// each way around 20 MB of input.  Here eight warps of the CTA gather every 128 x 32 tile of col straight from x into
// the 128-byte-swizzled shared-memory layout the tensor core reads (the layout a TMA box {32 k, 128 rows} would
// produce: row r at byte r * 128, its 16-byte chunk j stored at chunk position j ^ (r & 7)), together with the low
// part, while the weight tiles -- a plain K-major matrix -- arrive by TMA.  x is re-read KH*KW/S^2 times from L1 / L2,
// never from a materialised matrix.
//
// One CTA = 128 output pixels x BN output channels; warp 0 lane 0: TMA producer of the weight tiles; warp 1 lane 0: MMA
// issuer (TMEM accumulator, all of K in one pass: the truncating accumulation costs about 7.5e-9 * K relative error,
// so one CTA takes at most 576 of K; for longer reductions up to 2304 -- 256 channels x 3 x 3 -- the launcher starts
// clusters of two to four CTAs that split K and hand their partial tiles to the first one, one after the other, through
// distributed shared memory; still longer reductions go to the explicit path); warps 2..9:
// gather, then epilogue (bias / folded BatchNorm scale / ReLU / SiLU, NCHW store).  Two 48 KB (BN = 64) stages per CTA
// so that two CTAs share an SM and one's prologue and epilogue overlap the other's main loop.  Every wait is bounded.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstring>

#include "../../include/odl_b200.h"
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
constexpr int kBM       = 128;
constexpr int kBK       = 32;
constexpr int kUmmaK    = 8;
constexpr int kEpiWarps = 8;
constexpr int kThreads  = 64 + 32 * kEpiWarps;
constexpr int kStages   = 2;
constexpr int kAuxBytes = 256;
constexpr int kMaxK     = 576;                   // longest reduction one CTA keeps in TMEM (4.3e-6 of truncation error);
constexpr int kMaxCluster = 4;                   // a cluster of up to four CTAs splits longer ones: K <= 2304
constexpr int kPartOffset = 40960;               // where rank 1's partial tile lands in rank 0's dead operand ring (after
                                                 // the epilogue's transpose slabs: 8 warps x 32 x 36 floats)
constexpr int kTabBytes = (kMaxK + 32) * 8;      // per-k lookup table {offset, kh << 16 | kw}, padded to a K-block

struct IgemmGeom
{
    int N, C, H, W, KH, KW, S, P, OH, OW;
    int ckk;   // C*KH*KW = K of the GEMM
    int rows;  // N*OH*OW = M of the GEMM
};

template <int BN>
struct IgemmCfg
{
    static constexpr int a_bytes     = kBM * kBK * 4;
    static constexpr int b_bytes     = BN * kBK * 4;
    static constexpr int stage_bytes = 2 * (a_bytes + b_bytes);  // A, A_small, B, B_small
    static constexpr int smem_bytes  = 1024 + kStages * stage_bytes + kAuxBytes + kTabBytes;
    static constexpr int tmem_cols   = BN < 32 ? 32 : BN;
    static constexpr int warp_cols   = BN / 2;
};

template <int BN>
__global__ void __launch_bounds__(kThreads, 2)
conv_igemm_kernel(const __grid_constant__ TmapPack tm, const float *__restrict__ x, const IgemmGeom g, const GemmParams p,
                  const int terms, const int cluster_k)
{
    using Cfg = IgemmCfg<BN>;
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
        // (the two CTAs of a K-splitting cluster meet at cluster barriers: neither may leave early on its own)
        *early_out = (cluster_k == 1 && p.err != nullptr && *reinterpret_cast<volatile int *>(p.err) != 0) ? 1 : 0;
        *abort_f   = 0;
    }
    __syncthreads();
    if (*early_out)
        return;

    const int tiles_n = (p.N + BN - 1) / BN;
    const int tile_m  = blockIdx.x / tiles_n;
    const int tile_n  = blockIdx.x - tile_m * tiles_n;
    const int m0 = tile_m * kBM, n0 = tile_n * BN;
    // K-blocks [kb0, kb0 + num_kb) of the reduction belong to this CTA (all of them unless a cluster splits K)
    const int total_kb = (g.ckk + kBK - 1) / kBK;
    const int kb_per   = (total_kb + cluster_k - 1) / cluster_k;
    const int kb0      = blockIdx.y * kb_per;
    const int num_kb   = max(0, min(kb_per, total_kb - kb0));

    // Per-k table, built once per CTA: x[n, c, h0 + kh, w0 + kw] sits at pix_off + ktab[k].x with
    // ktab[k].x = (c * H + kh) * W + kw; ktab[k].y = kh << 16 | kw serves the bounds checks of border pixels.
    // Entries past C*KH*KW (the padding of the last K-block) are marked with y = -1.
    for (int kl = threadIdx.x; kl < num_kb * kBK; kl += kThreads)
    {
        int2 e      = make_int2(0, -1);
        const int k = kb0 * kBK + kl;
        if (k < g.ckk)
        {
            const int khw = g.KH * g.KW;
            const int c = k / khw, rm = k - c * khw, kh = rm / g.KW, kw = rm - kh * g.KW;
            e = make_int2((c * g.H + kh) * g.W + kw, (kh << 16) | kw);
        }
        ktab[kl] = e;
    }
    if (warp == 0 && lane == 0)
    {
        ptx::prefetch_tmap(&tm.b);
        if (terms == 3)
            ptx::prefetch_tmap(&tm.b_small);
        for (int s = 0; s < kStages; ++s)
        {
            ptx::mbar_init(&b_full[s], 1);
            ptx::mbar_init(&a_full[s], kEpiWarps);
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
        // ================================================================= TMA producer: weight tiles
        if (lane == 0)
        {
            int issued = 0;
            for (int kb = 0; kb < num_kb; ++kb)
            {
                const int s = kb % kStages;
                if (!ptx::mbar_wait_quiet(&empty_bar[s], ((kb / kStages) & 1) ^ 1, abort_f))
                    break;
                uint8_t *sb = tiles + s * Cfg::stage_bytes + 2 * Cfg::a_bytes;
                ptx::mbar_arrive_expect_tx(&b_full[s], Cfg::b_bytes * (terms == 3 ? 2 : 1));
                ptx::tma_load_2d(sb, &tm.b, &b_full[s], (kb0 + kb) * kBK, n0);
                if (terms == 3)
                    ptx::tma_load_2d(sb + Cfg::b_bytes, &tm.b_small, &b_full[s], (kb0 + kb) * kBK, n0);
                ++issued;
            }
            if (*abort_f)
            {
                const int first = issued > kStages ? issued - kStages : 0;
                for (int kb = first; kb < issued; ++kb)
                    ptx::mbar_wait_quiet(&b_full[kb % kStages], (kb / kStages) & 1, nullptr);
            }
        }
        __syncwarp();
        for (int r = 1; r < cluster_k; ++r)  // the barriers of the epilogue warps' hand-over below
        {
            ptx::cluster_sync();
            ptx::cluster_sync();
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
        __syncwarp();
        for (int r = 1; r < cluster_k; ++r)
        {
            ptx::cluster_sync();
            ptx::cluster_sync();
        }
    }
    else
    {
        // ================================================================= gather (im2col on the fly), then epilogue
        const int e    = warp - 2;
        const int q    = warp & 3;   // TMEM lane quarter this warp may read; also the 32-row group it gathers
        const int h    = e >> 2;     // half of the tile's columns (epilogue) / half of the K-block (gather)
        const int r    = 32 * q + lane;  // tile row gathered by this thread
        const int pix  = m0 + r;
        const bool row_ok = pix < g.rows;
        int n = 0, oh = 0, ow = 0;
        if (row_ok)
        {
            ow          = pix % g.OW;
            const int t = pix / g.OW;
            oh          = t % g.OH;
            n           = t / g.OH;
        }
        const int h0 = oh * g.S - g.P, w0 = ow * g.S - g.P;
        // 32-bit element offsets (the launcher keeps x below 2^31 elements)
        const int pix_off = (n * g.C * g.H + h0) * g.W + w0;
        // pixels whose whole window lies inside the image need no bounds checks
        const bool interior = row_ok && h0 >= 0 && h0 + g.KH <= g.H && w0 >= 0 && w0 + g.KW <= g.W;
        bool have           = true;
        // The 16 values of K-block kb are loaded into registers one K-block ahead of the stores: the loads need no
        // barrier (x is read-only), so their latency overlaps the previous block's stores, fence and hand-over.
        auto gather = [&](int kb, float (&v)[16]) {
            const int2 *tab = ktab + kb * kBK + 16 * h;  // this thread's 16 consecutive k (same for the whole warp)
            if (interior)
            {
#pragma unroll
                for (int i = 0; i < 16; ++i)
                {
                    const int2 e = tab[i];
                    v[i]         = e.y >= 0 ? __ldg(x + pix_off + e.x) : 0.f;
                }
            }
            else
            {
#pragma unroll
                for (int i = 0; i < 16; ++i)
                {
                    const int2 e  = tab[i];
                    const int hh  = h0 + (e.y >> 16), ww = w0 + (e.y & 0xffff);
                    const bool in = row_ok && e.y >= 0 && hh >= 0 && hh < g.H && ww >= 0 && ww < g.W;
                    v[i]          = in ? __ldg(x + pix_off + e.x) : 0.f;
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
            uint8_t *row_big   = tiles + s * Cfg::stage_bytes + r * 128;
            uint8_t *row_small = row_big + Cfg::a_bytes;
#pragma unroll
            for (int j4 = 0; j4 < 4; ++j4)
            {
                const int chunk = ((4 * h + j4) ^ (r & 7)) * 16;  // 128-byte swizzle: chunk index XOR row-in-atom
                *reinterpret_cast<float4 *>(row_big + chunk) = make_float4(v[4 * j4], v[4 * j4 + 1], v[4 * j4 + 2], v[4 * j4 + 3]);
                if (terms == 3)
                    *reinterpret_cast<float4 *>(row_small + chunk) =
                        make_float4(tf32_small(v[4 * j4]), tf32_small(v[4 * j4 + 1]), tf32_small(v[4 * j4 + 2]),
                                    tf32_small(v[4 * j4 + 3]));
            }
            ptx::fence_proxy_async_smem();  // generic-proxy writes -> visible to the tensor core's reads
            __syncwarp();
            if (lane == 0)
                ptx::mbar_arrive(&a_full[s]);
        }
        if (have && num_kb > 0)
            have = __all_sync(0xffffffffu, ptx::mbar_wait_quiet(acc_full, 0, abort_f));
        const int cw = h * Cfg::warp_cols;
        float acc[Cfg::warp_cols];
#pragma unroll
        for (int i = 0; i < Cfg::warp_cols; ++i)
            acc[i] = 0.f;
        if (have && num_kb > 0)
        {
            ptx::tc_fence_after_sync();
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
        }
        if (cluster_k > 1)
        {
            // K split over the CTAs of the cluster: ranks 1, 2, ... in turn write their partial tile into rank 0's dead
            // operand ring (one staging slot, layout [warp][column][lane]) and rank 0 adds it -- a fixed order -- then
            // runs the epilogue.  Two cluster barriers per rank: slot free / all MMAs done, and data visible.
            const uint32_t rank = ptx::cluster_ctarank();
            float *part         = stg_all + kPartOffset / 4 + static_cast<size_t>(e) * Cfg::warp_cols * 32;
            for (int r = 1; r < cluster_k; ++r)
            {
                __syncwarp();
                ptx::cluster_sync();
                if (static_cast<int>(rank) == r && have)
                {
                    const uint32_t dst = ptx::map_to_cta(ptx::smem_u32(part), 0);
#pragma unroll
                    for (int i = 0; i < Cfg::warp_cols; ++i)
                        ptx::st_shared_cluster_f32(dst + (i * 32 + lane) * 4, acc[i]);
                }
                ptx::cluster_sync();
                if (rank == 0)
                {
#pragma unroll
                    for (int i = 0; i < Cfg::warp_cols; ++i)
                        acc[i] += part[i * 32 + lane];
                }
            }
            if (rank != 0)
                have = false;
        }
        if (have)
            gemm_epilogue_store<BN, Cfg::warp_cols>(p, acc, stg_all + e * 32 * kStgLd, m0, n0, cw, q, lane);
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
int launch_igemm(const TmapPack &tm, const float *x, const IgemmGeom &g, const GemmParams &p, int terms, cudaStream_t stream)
{
    using Cfg = IgemmCfg<BN>;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    dev &= 63;
    if (!attr_set[dev])
    {
        cudaError_t e = cudaFuncSetAttribute(conv_igemm_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::smem_bytes);
        if (e != cudaSuccess)
        {
            set_last_error("cudaFuncSetAttribute(conv_igemm, smem=%d) failed: %s", Cfg::smem_bytes, cudaGetErrorString(e));
            return kCudaError;
        }
        attr_set[dev] = true;
    }
    const int tiles_m = (g.rows + kBM - 1) / kBM, tiles_n = (p.N + BN - 1) / BN;
    const int cluster_k = (g.ckk + kMaxK - 1) / kMaxK;  // 1..kMaxCluster (the caller checked eligibility)
    static_assert(kPartOffset + kBM * BN * 4 <= kStages * Cfg::stage_bytes, "rank 1's partial tile must fit the ring");
    cudaLaunchConfig_t cfg;
    std::memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim          = dim3(tiles_m * tiles_n, cluster_k, 1);
    cfg.blockDim         = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = Cfg::smem_bytes;
    cfg.stream           = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id               = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = cluster_k;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs                = attr;
    cfg.numAttrs             = cluster_k > 1 ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, conv_igemm_kernel<BN>, tm, x, g, p, terms, cluster_k);
    ++g_launch_count;
    if (e != cudaSuccess)
    {
        set_last_error("conv_igemm_kernel<%d> launch failed: %s", BN, cudaGetErrorString(e));
        return kCudaError;
    }
    return kOk;
}
}  // namespace

// Test hook: 0 = implicit GEMM / direct kernels where they apply, 1 = always the explicit im2col + GEMM paths,
// 2 = like 0 but without the direct weight-gradient kernel (small layers then take the implicit-GEMM one),
// 3 = like 0 but without the direct forward kernel (small layers then take the implicit-GEMM forward).
int g_conv_mode = 0;

bool conv_igemm_eligible(int64_t N, int64_t C, int64_t H, int64_t W, int64_t OC, int KH, int KW, int OH, int OW)
{
    const int64_t ckk = C * KH * KW, rows = N * OH * OW;
    return g_conv_mode != 1 && ckk <= kMaxCluster * kMaxK && OC <= 1024 && rows < (int64_t(1) << 31) - 256 && N * C * H * W < (int64_t(1) << 31) - (int64_t(1) << 20);
}

// w_big / w_small: the weights as a K-major [OC][ldw] matrix (ldw a multiple of 4, 16-byte aligned) and its low part.
int conv_igemm_launch(const float *x, const float *w_big, const float *w_small, int64_t ldw, const float *bias,
                      const float *scale, float *y, int64_t N, int64_t C, int64_t H, int64_t W, int64_t OC, int KH, int KW,
                      int S, int P, int OH, int OW, int act, int terms, cudaStream_t stream)
{
    IgemmGeom g;
    g.N = (int)N, g.C = (int)C, g.H = (int)H, g.W = (int)W, g.KH = KH, g.KW = KW, g.S = S, g.P = P, g.OH = OH, g.OW = OW;
    g.ckk  = (int)(C * KH * KW);
    g.rows = (int)(N * OH * OW);
    GemmParams p;
    std::memset(&p, 0, sizeof(p));
    p.D     = y;
    p.bias  = bias;
    p.scale = scale;
    p.err   = device_error_flag();
    p.M = g.rows, p.N = (int)OC, p.K = g.ckk;
    p.ldd   = (int)OC;
    p.flags = kEpiNCHW | (bias ? kEpiBias : 0) | (scale ? kEpiScale : 0) | (act == 1 ? kEpiRelu : 0) | (act == 2 ? kEpiSilu : 0);
    p.ohw   = OH * OW;
    const int bn = OC <= 64 ? 64 : 128;
    TmapPack tm;
    std::memset(&tm, 0, sizeof(tm));
    int rc;
    if ((rc = make_tmap(&tm.b, w_big, OC, g.ckk, ldw, kBK, bn, CU_TENSOR_MAP_SWIZZLE_128B)))
        return rc;
    if (terms == 3 && (rc = make_tmap(&tm.b_small, w_small, OC, g.ckk, ldw, kBK, bn, CU_TENSOR_MAP_SWIZZLE_128B)))
        return rc;
    return bn == 64 ? launch_igemm<64>(tm, x, g, p, terms, stream) : launch_igemm<128>(tm, x, g, p, terms, stream);
}

// ---- input gradient of a stride-1 convolution as a convolution: gx = conv(gy, Wf, pad K-1-P) with
//      Wf[c][oc][kh][kw] = W[oc][c][KH-1-kh][KW-1-kw].  This kernel writes Wf as the K-major [C][ldf] matrix the implicit
//      GEMM reads (pitch ldf >= OC*KH*KW, padding zeroed) together with its 3xTF32 low part.
namespace
{
__global__ void __launch_bounds__(256) conv_weight_flip_kernel(const float *__restrict__ w, float *__restrict__ wf,
                                                               float *__restrict__ wf_small, int OC, int C, int KH, int KW,
                                                               int ldf)
{
    const int c = blockIdx.y, kk = KH * KW;
    for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < ldf; j += gridDim.x * blockDim.x)
    {
        float v = 0.f;
        if (j < OC * kk)
        {
            const int oc = j / kk, t = j - oc * kk;
            v = __ldg(w + (static_cast<size_t>(oc) * C + c) * kk + (kk - 1 - t));  // both kernel axes reversed
        }
        wf[static_cast<size_t>(c) * ldf + j] = v;
        if (wf_small)
            wf_small[static_cast<size_t>(c) * ldf + j] = tf32_small(v);
    }
}
}  // namespace

bool conv_dx_igemm_eligible(int64_t N, int64_t C, int64_t H, int64_t W, int64_t OC, int KH, int KW, int S, int P, int OH,
                            int OW)
{
    return S == 1 && KH == KW && P <= KH - 1 && conv_igemm_eligible(N, OC, OH, OW, C, KH, KW, (int)H, (int)W);
}

// wf / wf_small: scratch of C * pad4(OC*KH*KW) floats each (wf_small may be null in plain TF32).
int conv_dx_igemm_launch(const float *gy, const float *w, float *wf, float *wf_small, float *gx, int64_t N, int64_t C,
                         int64_t H, int64_t W, int64_t OC, int KH, int KW, int P, int OH, int OW, int terms, cudaStream_t stream)
{
    const int ldf = static_cast<int>((OC * KH * KW + 3) & ~int64_t(3));
    conv_weight_flip_kernel<<<dim3((ldf + 255) / 256, (unsigned)C), 256, 0, stream>>>(w, wf, wf_small, (int)OC, (int)C, KH,
                                                                                       KW, ldf);
    ++g_launch_count;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
    {
        set_last_error("conv_weight_flip_kernel launch failed: %s", cudaGetErrorString(e));
        return kCudaError;
    }
    return conv_igemm_launch(gy, wf, wf_small, ldf, nullptr, nullptr, gx, N, OC, OH, OW, C, KH, KW, 1, KH - 1 - P, (int)H,
                             (int)W, 0, terms, stream);
}

}  // namespace odl

extern "C" int odl_debug_set_conv_mode(int mode)
{
    odl::g_conv_mode = mode;
    return 0;
}
