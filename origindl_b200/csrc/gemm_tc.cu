// tcgen05 / TMEM / TMA GEMM for sm_100a:  D[M,N] = A[M,K] * B[N,K]^T  in TF32 or 3xTF32, fp32 accumulate.
//
// One CTA computes one 128 x BN tile of D.  Warp roles (192 threads):
//   warp 0      TMA producer: one elected lane streams 128-byte-swizzled operand tiles into a ring of stages.
//   warp 1      TMEM owner and MMA issuer: one elected lane issues tcgen05.mma (kind::tf32, operands from
//               shared-memory descriptors, accumulator in TMEM) and commits stage-free / accumulator-ready barriers.
//   warps 2..5  epilogue: tcgen05.ld the accumulator (each warp owns the 32 TMEM lanes of its quarter), transpose
//               through a padded shared-memory slab, then apply bias / ReLU / ReLU-mask / column sums and write D
//               (and the low part of its TF32 split) with coalesced 128-bit stores.
//
// Operand majorness is a run-time property.  "K-major" means the reduction index is contiguous in memory
// (A stored [M][K], B stored [N][K]); "MN-major" means the M (or N) index is contiguous (A stored [K][M],
// B stored [K][N]).  Both are fed to the tensor core without a transpose pass:
//   K-major : one TMA box {32 k, rows} per tile -> rows x 128 B, SWIZZLE_128B; descriptor SBO = 1024 B,
//             each K=8 MMA step advances the start address by 32 B inside the swizzled row.
//   MN-major: boxes {32 mn, 32 k} (4 KB each) laid side by side, written with the 32-byte-chunk variant of the
//             128-byte swizzle (the only layout the tensor core accepts for MN-major 32-bit operands: its atom
//             is 4 k-rows x 128 B); descriptor LBO = 4096 B (next 32 mn), SBO = 512 B (next 4 k), each K=8 MMA
//             step advances the start address by 1024 B.
//
// 3xTF32: every operand X comes as two fp32 arrays, X itself (the tensor core reads its top 19 bits, i.e.
// trunc_tf32(X)) and X_small = tf32(X - trunc_tf32(X)); the accumulator receives
// A*B + A*B_small + A_small*B, which restores fp32-class accuracy (the dropped term is ~2^-22 relative).
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <mutex>

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

constexpr int kBM          = 128;  // rows of D per CTA == TMEM lanes == UMMA M
constexpr int kUmmaK       = 8;    // K per tcgen05.mma for kind::tf32
constexpr int kEpiWarps    = 8;    // two warps per TMEM lane quarter, each owning half of the tile's columns
constexpr int kThreads     = 64 + 32 * kEpiWarps;
constexpr int kGroupM      = 16;   // tile rasterisation: CTAs walk 16 row-tiles before moving to the next column-tile
constexpr int kSmemBudget  = 227 * 1024;
constexpr int kAuxBytes    = 1024;  // barriers, TMEM pointer, abort flag
constexpr int kPartOffset  = 40960; // split-K partial sums of cluster ranks 1.. start here in rank 0's ring (after the
                                    // epilogue's transpose slabs: 8 warps x 32 x 36 floats)
constexpr int kMaxStages   = 8;

// BK: fp32 elements of K per pipeline stage: 32 (128-byte swizzle rows) or 16 (64-byte rows, twice as many stages
// in flight for the same shared memory, which hides the load latency of the wide 3xTF32 stages).
template <int BN, int BK>
struct TileCfg
{
    static constexpr int a_bytes   = kBM * BK * 4;
    static constexpr int b_bytes   = BN * BK * 4;
    static constexpr int mn_box    = 32 * BK * 4;  // bytes of one {32 mn, BK k} box of an MN-major operand
    __host__ __device__ static constexpr int stage_bytes(int terms) { return (a_bytes + b_bytes) * (terms == 3 ? 2 : 1); }
    __host__ __device__ static constexpr int stages(int terms)
    {
        // the ring (>= 48 KB in every configuration) also hosts the 36 KB of epilogue transpose slabs afterwards
        int s = (kSmemBudget - 1024 /*alignment slack*/ - kAuxBytes) / stage_bytes(terms);
        return s > kMaxStages ? kMaxStages : s;
    }
    __host__ __device__ static constexpr int smem_bytes(int terms) { return 1024 + kAuxBytes + stages(terms) * stage_bytes(terms); }
    static constexpr int tmem_cols  = 2 * BN;  // two accumulators: the MMAs fill one while the other is drained
    static constexpr int warp_cols  = BN / 2;  // columns of the tile owned by one epilogue warp
};

// The accumulator is drained from TMEM into fp32 registers every `chunk_kb` K-blocks.  The tensor core adds into
// TMEM with truncation, which biases a long running sum towards zero by about 7.5e-9 * (chunk length in K) relative
// to the largest result; summing short chunks in registers (round-to-nearest) keeps 3xTF32 at fp32-class accuracy
// for any K.
template <int BN, int BK>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ TmapPack tm, const GemmParams p, const int a_mn, const int b_mn, const int terms,
               const int stages, const int chunk_kb, const int slabs, const int cluster_k)
{
    using Cfg = TileCfg<BN, BK>;
    extern __shared__ uint8_t smem_raw[];

    // ---- carve shared memory (tiles need 1024-byte alignment for the 128-byte swizzle)
    uint8_t *base = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    // A stage holds `slabs` K-slabs of BK elements each (2 in plain TF32 on the wide tile: twice the MMAs per stage
    // release, which is what bounds that mode); a "K-block" below is one stage, BK * slabs elements of K.
    const int slab_bytes  = Cfg::stage_bytes(terms);
    const int stage_bytes = slab_bytes * slabs;
    uint8_t *tiles        = base;
    float *stg_all        = reinterpret_cast<float *>(base);  // reused after the last MMA has read the ring
    uint8_t *aux_base     = base + stages * stage_bytes;
    uint64_t *full_bar    = reinterpret_cast<uint64_t *>(aux_base);
    uint64_t *empty_bar   = full_bar + kMaxStages;
    uint64_t *acc_full    = empty_bar + kMaxStages;  // [2]
    uint64_t *acc_empty   = acc_full + 2;            // [2]
    uint32_t *tmem_slot   = reinterpret_cast<uint32_t *>(acc_empty + 2);
    volatile int *abort_f = reinterpret_cast<volatile int *>(tmem_slot + 1);
    int *early_out        = const_cast<int *>(abort_f) + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    // ---- a launch that follows a timed-out one does nothing
    if (threadIdx.x == 0)
    {
        // (the CTAs of a split-K cluster meet at cluster barriers below, so none of them may leave early on its own
        // reading of the flag; their waits are bounded all the same)
        *early_out = (cluster_k == 1 && p.err != nullptr && *reinterpret_cast<volatile int *>(p.err) != 0) ? 1 : 0;
        *abort_f   = 0;
    }
    __syncthreads();
    if (*early_out)
        return;

    // ---- tile coordinates (grouped rasterisation for L2 reuse)
    const int tiles_m = (p.M + kBM - 1) / kBM;
    const int tiles_n = (p.N + BN - 1) / BN;
    int tile_m, tile_n;
    {
        const int per_group = kGroupM * tiles_n;
        const int g         = blockIdx.x / per_group;
        const int first_m   = g * kGroupM;
        const int gsz       = min(tiles_m - first_m, kGroupM);
        const int local     = blockIdx.x - g * per_group;
        tile_m              = first_m + local % gsz;
        tile_n              = local / gsz;
    }
    const int m0      = tile_m * kBM;
    const int n0      = tile_n * BN;
    const int kb_first = blockIdx.y * p.kb_per_split;  // split-K: this CTA reduces K-blocks [kb_first, kb_first + num_kb)
    const int num_kb   = min((p.K + BK * slabs - 1) / (BK * slabs) - kb_first, p.kb_per_split);
    const int nchunks  = (num_kb + chunk_kb - 1) / chunk_kb;

    // ---- one-time setup
    if (warp == 0 && lane == 0)
    {
        ptx::prefetch_tmap(&tm.a);
        ptx::prefetch_tmap(&tm.b);
        if (terms == 3)
        {
            ptx::prefetch_tmap(&tm.a_small);
            ptx::prefetch_tmap(&tm.b_small);
        }
        for (int s = 0; s < stages; ++s)
        {
            ptx::mbar_init(&full_bar[s], 1);
            ptx::mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; ++b)
        {
            ptx::mbar_init(&acc_full[b], 1);
            ptx::mbar_init(&acc_empty[b], kEpiWarps);
        }
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
        // ================================================================= TMA producer
        if (lane == 0)
        {
            int issued = 0;
            for (int kb = 0; kb < num_kb; ++kb)
            {
                const int s       = kb % stages;
                const uint32_t ph = (kb / stages) & 1;
                if (!ptx::mbar_wait(&empty_bar[s], ph ^ 1, abort_f))
                    break;
                ptx::mbar_arrive_expect_tx(&full_bar[s], stage_bytes);
                for (int sl = 0; sl < slabs; ++sl)
                {
                    uint8_t *st  = tiles + s * stage_bytes + sl * slab_bytes;
                    const int k0 = ((kb_first + kb) * slabs + sl) * BK;
                    for (int t = 0; t < (terms == 3 ? 2 : 1); ++t)
                    {
                        uint8_t *sa           = st + t * Cfg::a_bytes;
                        const CUtensorMap *ma = t ? &tm.a_small : &tm.a;
                        if (!a_mn)
                        {
                            ptx::tma_load_2d(sa, ma, &full_bar[s], k0, m0);
                        }
                        else if (a_mn & 2)
                        {
                            ptx::tma_load_3d(sa, ma, &full_bar[s], 0, k0, m0 / 32);  // all four 32 x BK boxes in one copy
                        }
                        else
                        {
    #pragma unroll
                            for (int j = 0; j < kBM / 32; ++j)
                                ptx::tma_load_2d(sa + j * Cfg::mn_box, ma, &full_bar[s], m0 + 32 * j, k0);
                        }
                }
                uint8_t *sb0 = st + (terms == 3 ? 2 : 1) * Cfg::a_bytes;
                for (int t = 0; t < (terms == 3 ? 2 : 1); ++t)
                {
                    uint8_t *sb           = sb0 + t * Cfg::b_bytes;
                    const CUtensorMap *mb = t ? &tm.b_small : &tm.b;
                    if (!b_mn)
                    {
                        ptx::tma_load_2d(sb, mb, &full_bar[s], k0, n0);
                    }
                    else if (b_mn & 2)
                    {
                        ptx::tma_load_3d(sb, mb, &full_bar[s], 0, k0, n0 / 32);
                    }
                    else
                    {
#pragma unroll
                        for (int j = 0; j < BN / 32; ++j)
                            ptx::tma_load_2d(sb + j * Cfg::mn_box, mb, &full_bar[s], n0 + 32 * j, k0);
                    }
                }
                }
                ++issued;
            }
            if (*abort_f)
            {
                // Gave up somewhere: let the copies already in flight land before the CTA's memory is released.
                const int first = issued > stages ? issued - stages : 0;
                for (int kb = first; kb < issued; ++kb)
                    ptx::mbar_wait(&full_bar[kb % stages], (kb / stages) & 1, nullptr);
            }
        }
        if (cluster_k > 1)
        {
            __syncwarp();
            ptx::cluster_sync();
            ptx::cluster_sync();
        }
    }
    else if (warp == 1)
    {
        // ================================================================= MMA issuer
        if (lane == 0)
        {
            const uint32_t idesc  = ptx::make_idesc_tf32(kBM, BN, a_mn != 0, b_mn != 0);
            const uint32_t a_step = a_mn ? 1024u : 32u;  // bytes per K=8 step
            const uint32_t b_step = b_mn ? 1024u : 32u;
            // K-major: 8-row groups of (BK*4)-byte rows; MN-major: 32-mn groups one box apart, 4-k groups 512 B apart
            constexpr uint32_t k_sbo = 8u * BK * 4u;
            constexpr uint32_t k_lay = BK == 32 ? ptx::kLayoutSw128 : ptx::kLayoutSw64;
            const uint32_t a_lbo  = a_mn ? Cfg::mn_box : 16u;
            const uint32_t b_lbo  = b_mn ? Cfg::mn_box : 16u;
            const uint32_t a_sbo  = a_mn ? 512u : k_sbo;
            const uint32_t b_sbo  = b_mn ? 512u : k_sbo;
            const uint32_t a_lay  = a_mn ? ptx::kLayoutSw128Base32 : k_lay;
            const uint32_t b_lay  = b_mn ? ptx::kLayoutSw128Base32 : k_lay;
            bool ok               = true;
            int kb                = 0;
            for (int c = 0; c < nchunks && ok; ++c)
            {
                const int buf        = c & 1;
                const uint32_t use   = static_cast<uint32_t>(c >> 1);
                const uint32_t tmem_d = tmem_base + buf * BN;
                if (!ptx::mbar_wait(&acc_empty[buf], (use & 1) ^ 1, abort_f))
                {
                    ok = false;
                    break;
                }
                ptx::tc_fence_after_sync();
                const int kb_end = min(kb + chunk_kb, num_kb);
                for (bool first = true; kb < kb_end; ++kb)
                {
                    const int s       = kb % stages;
                    const uint32_t ph = (kb / stages) & 1;
                    if (!ptx::mbar_wait(&full_bar[s], ph, abort_f))
                    {
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after_sync();
                    for (int sl = 0; sl < slabs; ++sl)
                    {
                        const uint32_t sa  = ptx::smem_u32(tiles + s * stage_bytes + sl * slab_bytes);
                        const uint32_t sas = sa + Cfg::a_bytes;
                        const uint32_t sb  = sa + (terms == 3 ? 2 : 1) * Cfg::a_bytes;
                        const uint32_t sbs = sb + Cfg::b_bytes;
    #pragma unroll
                        for (int kk = 0; kk < BK / kUmmaK; ++kk)
                        {
                            const uint64_t da = ptx::make_smem_desc(sa + kk * a_step, a_lbo, a_sbo, a_lay);
                            const uint64_t db = ptx::make_smem_desc(sb + kk * b_step, b_lbo, b_sbo, b_lay);
                            if (terms == 3)
                            {
                                const uint64_t das = ptx::make_smem_desc(sas + kk * a_step, a_lbo, a_sbo, a_lay);
                                const uint64_t dbs = ptx::make_smem_desc(sbs + kk * b_step, b_lbo, b_sbo, b_lay);
                                // small cross terms first, the dominant term last
                                ptx::mma_tf32_ss(tmem_d, das, db, idesc, first ? 0u : 1u);
                                ptx::mma_tf32_ss(tmem_d, da, dbs, idesc, 1);
                                ptx::mma_tf32_ss(tmem_d, da, db, idesc, 1);
                            }
                            else
                            {
                                ptx::mma_tf32_ss(tmem_d, da, db, idesc, first ? 0u : 1u);
                            }
                            first = false;
                    }
                    }
                    ptx::mma_commit(&empty_bar[s]);  // stage reusable once these MMAs have read it
                }
                if (ok)
                    ptx::mma_commit(&acc_full[buf]);  // this chunk's accumulator is complete
            }
        }
        if (cluster_k > 1)
        {
            __syncwarp();
            ptx::cluster_sync();
            ptx::cluster_sync();
        }
    }
    else
    {
        // ================================================================= accumulate + epilogue (warps 2..9)
        const int e  = warp - 2;
        const int q  = warp & 3;                      // TMEM lane quarter this warp may read
        const int h  = e >> 2;                        // which half of the tile's columns
        const int cw = h * Cfg::warp_cols;            // first column owned by this warp
        float acc[Cfg::warp_cols];
        bool have = true;
        for (int c = 0; c < nchunks; ++c)
        {
            const int buf      = c & 1;
            const uint32_t use = static_cast<uint32_t>(c >> 1);
            have = __all_sync(0xffffffffu, ptx::mbar_wait(&acc_full[buf], use & 1, abort_f));
            if (!have)
                break;
            ptx::tc_fence_after_sync();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(32 * q) << 16) + buf * BN + cw;
#pragma unroll
            for (int j = 0; j < Cfg::warp_cols / 32; ++j)
            {
                uint32_t r[32];
                ptx::tmem_ld_32x32(taddr + 32 * j, r);
                ptx::tmem_ld_wait();
                if (c == 0)
                {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        acc[32 * j + i] = __uint_as_float(r[i]);
                }
                else
                {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        acc[32 * j + i] += __uint_as_float(r[i]);
                }
            }
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0)
                ptx::mbar_arrive(&acc_empty[buf]);
        }
        if (nchunks <= 0)
        {
#pragma unroll
            for (int i = 0; i < Cfg::warp_cols; ++i)
                acc[i] = 0.f;
        }
        if (cluster_k > 1)
        {
            // Split-K inside a thread-block cluster: the cluster_k CTAs along gridDim.y hold partial sums of the same
            // tile in registers.  Ranks 1.. write theirs into rank 0's (dead) operand ring through distributed shared
            // memory; rank 0 adds them in rank order -- the same bits every run -- and runs the normal epilogue, so
            // every epilogue flag works with this kind of split.  Layout [rank-1][warp][column][lane]: consecutive
            // lanes write consecutive words.
            __syncwarp();
            ptx::cluster_sync();  // every CTA of the cluster is past its last MMA: all operand rings are dead
            const uint32_t rank = ptx::cluster_ctarank();
            float *part         = stg_all + kPartOffset / 4;
            if (rank != 0 && have)
            {
                const uint32_t dst = ptx::map_to_cta(
                    ptx::smem_u32(part + (static_cast<size_t>(rank - 1) * kEpiWarps + e) * Cfg::warp_cols * 32), 0);
#pragma unroll
                for (int i = 0; i < Cfg::warp_cols; ++i)
                    ptx::st_shared_cluster_f32(dst + (i * 32 + lane) * 4, acc[i]);
            }
            ptx::cluster_sync();  // release / acquire: the partial sums are visible to rank 0
            if (rank == 0)
            {
                for (int r = 1; r < cluster_k; ++r)
                {
                    const float *src = part + (static_cast<size_t>(r - 1) * kEpiWarps + e) * Cfg::warp_cols * 32 + lane;
#pragma unroll
                    for (int i = 0; i < Cfg::warp_cols; ++i)
                        acc[i] += src[i * 32];
                }
            }
            else
            {
                have = false;  // only rank 0 stores the tile
            }
        }
        if (have)
        {
            // The last acc_full has fired, so every MMA has completed and every tile load was consumed: the operand
            // ring is dead and its first bytes now serve as per-warp transpose slabs (disjoint between warps).
            gemm_epilogue_store<BN, Cfg::warp_cols>(p, acc, stg_all + e * 32 * kStgLd, m0, n0, cw, q, lane);
        }
        ptx::tc_fence_before_sync();
    }

    // ---- teardown: everyone is done with TMEM before warp 1 releases it
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

// ---------------------------------------------------------------------------------------------- host side
}  // namespace
extern int g_chunk_kb;
extern int g_split_k;
extern int g_bk_override;
// Second pass of split-K: D[m][n] = sum over splits z (ascending) of slices[z][m][n].
__global__ void __launch_bounds__(256) splitk_sum_kernel(const float *__restrict__ slices, int splits, int M, int N, int lds,
                                                         float *__restrict__ D, int ldd)
{
    const int64_t total  = static_cast<int64_t>(M) * N;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const size_t slice   = static_cast<size_t>(M) * lds;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride)
    {
        const int m = static_cast<int>(i / N), n = static_cast<int>(i - static_cast<int64_t>(m) * N);
        const float *sp = slices + static_cast<size_t>(m) * lds + n;
        float s         = __ldcg(sp);
        for (int z = 1; z < splits; ++z)
            s += __ldcg(sp + z * slice);
        D[static_cast<size_t>(m) * ldd + n] = s;
    }
}

int splitk_sum_launch(const float *slices, int splits, int M, int N, int lds, float *D, int ldd, cudaStream_t stream)
{
    const int64_t total = static_cast<int64_t>(M) * N;
    splitk_sum_kernel<<<static_cast<unsigned>(std::min<int64_t>((total + 255) / 256, 148 * 8)), 256, 0, stream>>>(
        slices, splits, M, N, lds, D, ldd);
    ++g_launch_count;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
    {
        set_last_error("splitk_sum_kernel launch failed: %s", cudaGetErrorString(e));
        return kCudaError;
    }
    return kOk;
}

extern int g_slabs;
namespace
{
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn()
{
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    });
    return fn;
}

}  // namespace

// Tensor map over a row-major fp32 matrix with `rows` rows of `cols` contiguous elements (row pitch ld elements).
int make_tmap(CUtensorMap *out, const float *ptr, int64_t rows, int64_t cols, int64_t ld, int box_cols, int box_rows,
              CUtensorMapSwizzle swizzle)
{
    EncodeTiledFn fn = get_encode_fn();
    if (!fn)
    {
        set_last_error("cuTensorMapEncodeTiled entry point not available");
        return kCudaError;
    }
    cuuint64_t dims[2]    = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 4};
    cuuint32_t box[2]     = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
    cuuint32_t estr[2]    = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
    {
        set_last_error("cuTensorMapEncodeTiled failed: code %d (rows=%lld cols=%lld ld=%lld box=%dx%d ptr=%p)", (int)r,
                       (long long)rows, (long long)cols, (long long)ld, box_cols, box_rows, (const void *)ptr);
        return kCudaError;
    }
    return kOk;
}

int make_tmap_mn3d(CUtensorMap *out, const float *ptr, int64_t k_rows, int64_t mn_cols, int64_t ld, int box_k, int boxes,
                   CUtensorMapSwizzle swizzle)
{
    EncodeTiledFn fn = get_encode_fn();
    if (!fn || (mn_cols & 31))
        return kCudaError;  // the caller falls back to separate 2-D copies
    cuuint64_t dims[3]    = {32, static_cast<cuuint64_t>(k_rows), static_cast<cuuint64_t>(mn_cols / 32)};
    cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld) * 4, 128};
    cuuint32_t box[3]     = {32, static_cast<cuuint32_t>(box_k), static_cast<cuuint32_t>(boxes)};
    cuuint32_t estr[3]    = {1, 1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float *>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? kOk : kCudaError;
}

namespace
{
template <int BN, int BK>
int launch_bn(const TmapPack &tm, const GemmParams &p, int a_mn, int b_mn, int terms, cudaStream_t stream)
{
    using Cfg        = TileCfg<BN, BK>;
    // plain TF32 on the wide tile: two K-slabs per stage when the reduction is long enough to fill the ring
    int slabs = (terms == 1 && BN == 256 && BK == 32 && p.K >= 8 * BK) ? 2 : 1;
    if (g_slabs == 1 || g_slabs == 2)
        slabs = (terms == 1 && BK == 32) ? g_slabs : 1;
    const int stages = Cfg::stages(terms) / slabs;
    const int smem   = Cfg::smem_bytes(terms);
    static bool attr_set[64] = {};  // one flag per device for THIS instantiation
    int dev = 0;
    cudaGetDevice(&dev);
    dev &= 63;
    if (!attr_set[dev])
    {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, BK>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             Cfg::smem_bytes(1) > Cfg::smem_bytes(3) ? Cfg::smem_bytes(1)
                                                                                     : Cfg::smem_bytes(3));
        if (e != cudaSuccess)
        {
            set_last_error("cudaFuncSetAttribute(smem=%d) failed: %s", smem, cudaGetErrorString(e));
            return kCudaError;
        }
        attr_set[dev] = true;
    }
    const int tiles_m = (p.M + kBM - 1) / kBM;
    const int tiles_n = (p.N + BN - 1) / BN;
    const int num_kb   = (p.K + BK * slabs - 1) / (BK * slabs);  // in stages
    // Split-K when the output has too few tiles to fill 148 SMs.  Two forms:
    //  * inside a thread-block cluster of 2 or 4 CTAs along K (partial tiles combined through distributed shared
    //    memory in rank order by the CTA that then runs the epilogue): any epilogue, no scratch, no second launch --
    //    what small-batch layers need, whose CTAs are bound by how fast ONE SM can stream its K range;
    //  * across more CTAs than a cluster's staging area holds (long reductions into tiny outputs, plain epilogue
    //    only): every split stores its partial tile into a slice of a scratch buffer, a second pass adds the slices.
    // Both add in a fixed order.  g_split_k (test hook): 1 = never split, n > 1 = n slices, -n = cluster of n.
    GemmParams q = p;
    int splits = 1, cluster_k = 1;
    const int tiles = tiles_m * tiles_n;
    // rank 0 stages (cluster_k - 1) partial tiles of 128 x BN floats behind the transpose slabs of its dead operand ring
    const int ring       = stages * Cfg::stage_bytes(terms) * slabs;
    const int max_cluster = ring >= kPartOffset + 3 * kBM * BN * 4 ? 4 : (ring >= kPartOffset + kBM * BN * 4 ? 2 : 1);
    if (g_split_k != 1 && tiles * 2 <= 148)
    {
        int want = g_split_k > 1 ? g_split_k : 148 / tiles;
        if (g_split_k == 0 && want > num_kb / 4)
            want = num_kb / 4;  // at least four K-blocks per split
        const bool slices_ok = p.flags == 0 && num_kb * slabs >= 32;
        if (g_split_k < 0)
            cluster_k = -g_split_k <= max_cluster ? -g_split_k : max_cluster;
        else if (g_split_k > 1 || (slices_ok && want > max_cluster))
        {
            splits = want;
            if (g_split_k == 0 && splits > num_kb / 8)
                splits = num_kb / 8;
            if (splits < 1)
                splits = 1;
        }
        else if (want >= 2)
            cluster_k = (want >= 4 && max_cluster >= 4) ? 4 : (max_cluster >= 2 ? 2 : 1);
    }
    if (cluster_k > 1)
    {
        q.kb_per_split = (num_kb + cluster_k - 1) / cluster_k;
    }
    else
    {
        q.kb_per_split = (num_kb + splits - 1) / splits;
        splits         = (num_kb + q.kb_per_split - 1) / q.kb_per_split;
    }
    if (splits > 1)
    {
        q.flags |= kEpiSplitK;
        q.ldd = (p.N + 3) & ~3;
        q.D   = colsum_partial_scratch(splits * p.M, q.ldd);
        if (!q.D)
            return kCudaError;
    }
    int chunk_kb       = g_chunk_kb > 0 ? (g_chunk_kb + slabs - 1) / slabs : (terms == 3 ? 64 / BK : q.kb_per_split);
    if (chunk_kb > q.kb_per_split)
        chunk_kb = q.kb_per_split;
    cudaLaunchConfig_t cfg;
    std::memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim          = dim3(tiles, cluster_k > 1 ? cluster_k : splits, 1);
    cfg.blockDim         = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream           = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id               = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = cluster_k;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs                = attr;
    cfg.numAttrs             = cluster_k > 1 ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc_kernel<BN, BK>, tm, q, a_mn, b_mn, terms, stages, chunk_kb, slabs, cluster_k);
    ++g_launch_count;
    if (e != cudaSuccess)
    {
        set_last_error("gemm_tc_kernel<%d,%d> launch failed: %s", BN, BK, cudaGetErrorString(e));
        return kCudaError;
    }
    if (splits > 1)
        return splitk_sum_launch(q.D, splits, p.M, p.N, q.ldd, p.D, p.ldd, stream);
    return kOk;
}

}  // namespace

// Test hook: K-blocks accumulated in TMEM between two drains into registers; 0 = default
// (64 K elements, i.e. 2 blocks of 32, for 3xTF32; the whole K for plain TF32).
int g_chunk_kb = 0;
// Test hook: K-slabs of 32 per pipeline stage in plain TF32 (0 = automatic, 1 or 2).
int g_slabs = 0;
// Test hook: 0 = automatic split-K, 1 = never split, n > 1 = force n splits where the epilogue allows it.
int g_split_k = 0;
// Test hook: K elements per pipeline stage of the 256-wide tile (16 or 32; 0 = automatic).
int g_bk_override = 0;

// A / B operands must already satisfy the tiled-load rules (16-byte aligned base, ld % 4 == 0); the callers in
// linear.cu stage anything else through padded scratch.  a_mn / b_mn: 0 = K-major storage, 1 = MN-major storage.
int gemm_tc_launch(const float *A, const float *A_small, int64_t lda, int a_mn, const float *B, const float *B_small,
                   int64_t ldb, int b_mn, const GemmParams &p, int terms, int bn_hint, cudaStream_t stream)
{
    if (p.M <= 0 || p.N <= 0 || p.K <= 0 || !A || !B || !p.D || (terms != 1 && terms != 3))
    {
        set_last_error("gemm: invalid argument (M=%d N=%d K=%d terms=%d)", p.M, p.N, p.K, terms);
        return kInvalidArgument;
    }
    if (terms == 3 && (!A_small || !B_small))
    {
        set_last_error("gemm: 3xTF32 needs the low parts of both operands");
        return kInvalidArgument;
    }
    auto misaligned = [](const void *ptr, int64_t ld) { return (reinterpret_cast<uintptr_t>(ptr) & 15) || (ld & 3); };
    if (misaligned(A, lda) || misaligned(B, ldb) || (terms == 3 && (misaligned(A_small, lda) || misaligned(B_small, ldb))))
    {
        set_last_error("gemm: operand violates the 16-byte rule (lda=%lld ldb=%lld)", (long long)lda, (long long)ldb);
        return kMisaligned;
    }
    int bn = bn_hint;
    if ((p.flags & kEpiNCHW) && bn == 256)
        bn = 128;
    if (bn != 64 && bn != 128 && bn != 256)
    {
        // Pick the tile width with a small cost model fitted to measurements on B200.  One K-block (32 of K) costs a
        // CTA nearly the same time whatever the tile width -- 0.94 / 0.98 / 1.27 us for 64 / 128 / 256 columns in 3xTF32
        // (the A operand's shared-memory reads and the MMA issue do not shrink with N) -- so the widest tile is by far
        // the most efficient per SM, and a machine that a wide tiling leaves half empty is filled by splitting K over
        // a cluster (launch_bn) rather than by narrower tiles.  time = waves * (K-blocks per CTA * t_kb + fixed costs).
        const int tm           = (p.M + kBM - 1) / kBM;
        const int64_t k_blocks = (p.K + 31) / 32;
        const int64_t tiles256 = static_cast<int64_t>(tm) * ((p.N + 255) / 256);
        if (p.N > 128 && p.flags == 0 && tiles256 * 2 <= 148 && k_blocks >= 64)
        {
            bn = 256;  // long reduction, few tiles, plain epilogue (dW of a skinny layer): wide tiles + many K slices
        }
        else
        {
            static const int widths[3]    = {256, 128, 64};
            static const double t_kb3[3]  = {1.27, 0.98, 0.94}, t_kb1[3] = {0.60, 0.50, 0.45};
            static const double fixed[3]  = {14.0, 8.0, 6.0};
            static const int max_clus[3]  = {2, 2, 4};
            double best = 1e30;
            for (int i = 0; i < 3; ++i)
            {
                const int w = widths[i];
                if ((w == 256 && ((p.flags & kEpiNCHW) || p.N <= 128)) || (w == 128 && p.N <= 64))
                    continue;
                const int64_t tiles = static_cast<int64_t>(tm) * ((p.N + w - 1) / w);
                int c = 1;
                if (tiles * 2 <= 148)
                {
                    const int64_t want = std::min<int64_t>(148 / tiles, k_blocks / 4);
                    c = (want >= 4 && max_clus[i] >= 4) ? 4 : (want >= 2 ? 2 : 1);
                }
                const double waves = static_cast<double>((tiles * c + 147) / 148);
                const double t = waves * (static_cast<double>((k_blocks + c - 1) / c) * (terms == 3 ? t_kb3[i] : t_kb1[i]) +
                                          fixed[i] + (c > 1 ? 5.0 : 0.0));
                if (t < best)
                {
                    best = t;
                    bn   = w;
                }
            }
        }
    }
    if (gemm_pair_eligible(p, bn, a_mn, b_mn, terms))
        return gemm_pair_launch(A, A_small, lda, a_mn, B, B_small, ldb, b_mn, p, terms, stream);
    TmapPack tm;
    std::memset(&tm, 0, sizeof(tm));
    int rc;
    // A: K-major -> matrix [M][K], box {32, 128};  MN-major -> matrix [K][M], box {32, 32}
    // pipeline K-depth: BK = 32 everywhere.  BK = 16 (four 48 KB stages instead of two 96 KB ones for the 256-wide
    // 3xTF32 tile) was measured 5-40 % slower on B200: the loads are bound by the number of 128-byte-or-narrower rows
    // the TMA unit moves per cycle, not by bytes in flight, and halving the row width doubles the row count.
    int bk = 32;
    if (g_bk_override == 16 || g_bk_override == 32)
        bk = g_bk_override;
    if (bk == 16 && bn != 256)
        bk = 32;
    // MN-major operands whose extent is a multiple of 32: one 3-D copy per operand and K-slab instead of one 2-D copy
    // per 32 x BK box
    {
        CUtensorMap probe;
        if (a_mn && make_tmap_mn3d(&probe, A, p.K, p.M, lda, bk, kBM / 32, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B) == kOk)
            a_mn |= 2;
        if (b_mn && make_tmap_mn3d(&probe, B, p.K, p.N, ldb, bk, bn / 32, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B) == kOk)
            b_mn |= 2;
    }
    auto mk = [&](CUtensorMap *m, const float *ptr, int64_t ld, int mn, int64_t extent_mn, int box_rows_kmajor) {
        if (mn & 2)
            return make_tmap_mn3d(m, ptr, p.K, extent_mn, ld, bk, box_rows_kmajor / 32, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
        return mn ? make_tmap(m, ptr, p.K, extent_mn, ld, 32, bk, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B)
                  : make_tmap(m, ptr, extent_mn, p.K, ld, bk, box_rows_kmajor,
                              bk == 32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B);
    };
    if ((rc = mk(&tm.a, A, lda, a_mn, p.M, kBM)))
        return rc;
    if ((rc = mk(&tm.b, B, ldb, b_mn, p.N, bn)))
        return rc;
    if (terms == 3)
    {
        if ((rc = mk(&tm.a_small, A_small, lda, a_mn, p.M, kBM)))
            return rc;
        if ((rc = mk(&tm.b_small, B_small, ldb, b_mn, p.N, bn)))
            return rc;
    }
    switch (bn)
    {
        case 64:
            return launch_bn<64, 32>(tm, p, a_mn, b_mn, terms, stream);
        case 128:
            return launch_bn<128, 32>(tm, p, a_mn, b_mn, terms, stream);
        default:
            return bk == 16 ? launch_bn<256, 16>(tm, p, a_mn, b_mn, terms, stream)
                            : launch_bn<256, 32>(tm, p, a_mn, b_mn, terms, stream);
    }
}

}  // namespace odl
