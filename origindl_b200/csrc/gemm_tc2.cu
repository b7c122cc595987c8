// 2-CTA variant of the tcgen05 GEMM (tcgen05 cta_group::2): a pair of CTAs on neighbouring SMs computes one
// 256 x BN tile of D.  Each CTA keeps its own 128 rows of A and HALF of the B tile in shared memory and its own 128
// accumulator rows in TMEM; one thread of the pair's leader issues MMAs with M = 256 that read both CTAs' shared
// memory.  Per SM this halves the B bytes the TMA unit has to land per MMA cycle -- the measured limiter of the 1-CTA
// kernel -- and leaves room for a third 3xTF32 stage (64 KB per stage and CTA instead of 96 KB).
//
// Protocol inside a pair (cluster of 2; rank 0 = leader), all with plain mbarriers.  No load is multicast: every CTA
// issues its own tiled copies into its own shared memory.  The one cluster-wide instruction is the leader's
// tcgen05.commit with a CTA mask, which signals a barrier in both CTAs and moves no data.
//   full[s]      lives in the leader; the leader's producer arms it with the bytes of BOTH CTAs, both producers' TMA
//                loads report to it (the peer through the barrier's shared::cluster address);
//   empty[s]     one per CTA; the leader's MMA thread commits to its own and to the peer's after the MMAs of stage s;
//   acc_full[b]  one per CTA; committed to both when a chunk of K has been accumulated into TMEM buffer b;
//   acc_empty[b] lives in the leader; the 8 epilogue warps of each CTA arrive on it after draining buffer b.
// Everything else (operand layouts and descriptors, 3xTF32 terms, accumulator drains, epilogue) is the 1-CTA design.
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

constexpr int kBM         = 128;  // rows of D per CTA
constexpr int kBK         = 32;
constexpr int kUmmaK      = 8;
constexpr int kEpiWarps   = 8;
constexpr int kThreads    = 64 + 32 * kEpiWarps;
constexpr int kGroupM     = 8;    // rasterisation: 8 row-tiles of 256 per group
constexpr int kSmemBudget = 227 * 1024;
constexpr int kAuxBytes   = 1024;
constexpr int kMaxStages  = 8;

template <int BN>
struct PairCfg
{
    static constexpr int a_bytes  = kBM * kBK * 4;
    static constexpr int b_bytes  = (BN / 2) * kBK * 4;  // this CTA's half of the B tile
    static constexpr int mn_box   = 32 * kBK * 4;
    __host__ __device__ static constexpr int stage_bytes(int terms) { return (a_bytes + b_bytes) * (terms == 3 ? 2 : 1); }
    __host__ __device__ static constexpr int stages(int terms)
    {
        int s = (kSmemBudget - 1024 - kAuxBytes) / stage_bytes(terms);
        return s > kMaxStages ? kMaxStages : s;
    }
    __host__ __device__ static constexpr int smem_bytes(int terms) { return 1024 + kAuxBytes + stages(terms) * stage_bytes(terms); }
    static constexpr int tmem_cols = 2 * BN;
    static constexpr int warp_cols = BN / 2;
};

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc2_kernel(const __grid_constant__ TmapPack tm, const GemmParams p, const int a_mn, const int b_mn, const int terms,
                const int stages, const int chunk_kb, const int slabs)
{
    using Cfg = PairCfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *base = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    // `slabs` K-slabs of kBK elements per stage (2 in plain TF32: twice the MMAs per stage release)
    const int slab_bytes  = Cfg::stage_bytes(terms);
    const int stage_bytes = slab_bytes * slabs;
    uint8_t *tiles        = base;
    float *stg_all        = reinterpret_cast<float *>(base);
    uint8_t *aux_base     = base + stages * stage_bytes;
    uint64_t *full_bar    = reinterpret_cast<uint64_t *>(aux_base);
    uint64_t *empty_bar   = full_bar + kMaxStages;
    uint64_t *acc_full    = empty_bar + kMaxStages;
    uint64_t *acc_empty   = acc_full + 2;
    uint32_t *tmem_slot   = reinterpret_cast<uint32_t *>(acc_empty + 2);
    volatile int *abort_f = reinterpret_cast<volatile int *>(tmem_slot + 1);
    int *early_out        = const_cast<int *>(abort_f) + 1;

    const int warp      = threadIdx.x >> 5;
    const int lane      = threadIdx.x & 31;
    const uint32_t rank = ptx::cluster_ctarank();
    const bool leader   = rank == 0;

    if (threadIdx.x == 0)
    {
        *early_out = (leader && p.err != nullptr && *reinterpret_cast<volatile int *>(p.err) != 0) ? 1 : 0;
        *abort_f   = 0;
    }
    __syncthreads();
    ptx::cluster_sync();
    // A launch that follows a timed-out one does no work.  The LEADER reads the device flag and its peer takes the
    // leader's answer, so both CTAs of a pair always agree (a pair that disagreed could wait for each other in the
    // collective TMEM allocation); both still walk through every cluster barrier below.
    const bool skip = ptx::ld_shared_cluster_u32(ptx::map_to_cta(ptx::smem_u32(early_out), 0)) != 0;

    // ---- tile coordinates: blockIdx.x = 2 * pair + rank
    const int tiles_m = (p.M + 2 * kBM - 1) / (2 * kBM);
    const int tiles_n = (p.N + BN - 1) / BN;
    int tile_m, tile_n;
    {
        const int pair      = blockIdx.x >> 1;
        const int per_group = kGroupM * tiles_n;
        const int g         = pair / per_group;
        const int first_m   = g * kGroupM;
        const int gsz       = min(tiles_m - first_m, kGroupM);
        const int local     = pair - g * per_group;
        tile_m              = first_m + local % gsz;
        tile_n              = local / gsz;
    }
    const int m0      = tile_m * 2 * kBM + static_cast<int>(rank) * kBM;  // this CTA's rows of A and D
    const int n0      = tile_n * BN;                                      // the pair's columns of D
    const int nb0     = n0 + static_cast<int>(rank) * (BN / 2);           // this CTA's rows of the B tile
    const int num_kb  = (p.K + kBK * slabs - 1) / (kBK * slabs);  // stages
    const int nchunks = (num_kb + chunk_kb - 1) / chunk_kb;

    if (!skip)
    {
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
                ptx::mbar_init(&acc_empty[b], 2 * kEpiWarps);  // the epilogue warps of both CTAs
            }
            ptx::fence_mbar_init();
        }
        if (warp == 1)
        {
            ptx::tmem_alloc_pair(tmem_slot, Cfg::tmem_cols);
            ptx::tmem_relinquish_pair();
        }
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::cluster_sync();  // both CTAs' barriers exist before anyone signals across the pair
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = skip ? 0u : *tmem_slot;

    if (skip)
    {
        // nothing
    }
    else if (warp == 0)
    {
        // ================================================================= TMA producer (both CTAs)
        if (lane == 0)
        {
            int issued = 0;
            for (int kb = 0; kb < num_kb; ++kb)
            {
                const int s       = kb % stages;
                const uint32_t ph = (kb / stages) & 1;
                if (!ptx::mbar_wait(&empty_bar[s], ph ^ 1, abort_f))
                    break;
                if (leader)
                    ptx::mbar_arrive_expect_tx(&full_bar[s], 2 * stage_bytes);
                const uint32_t bar = ptx::map_to_cta(ptx::smem_u32(&full_bar[s]), 0);
                for (int sl = 0; sl < slabs; ++sl)
                {
                    uint8_t *st  = tiles + s * stage_bytes + sl * slab_bytes;
                    const int k0 = (kb * slabs + sl) * kBK;
                    for (int t = 0; t < (terms == 3 ? 2 : 1); ++t)
                    {
                        uint8_t *sa           = st + t * Cfg::a_bytes;
                        const CUtensorMap *ma = t ? &tm.a_small : &tm.a;
                        if (!a_mn)
                        {
                            ptx::tma_load_2d_pair(sa, ma, bar, k0, m0);
                        }
                        else if (a_mn & 2)
                        {
                            ptx::tma_load_3d_pair(sa, ma, bar, 0, k0, m0 / 32);  // all four 32 x 32 boxes in one copy
                        }
                        else
                        {
    #pragma unroll
                            for (int j = 0; j < kBM / 32; ++j)
                                ptx::tma_load_2d_pair(sa + j * Cfg::mn_box, ma, bar, m0 + 32 * j, k0);
                        }
                }
                uint8_t *sb0 = st + (terms == 3 ? 2 : 1) * Cfg::a_bytes;
                for (int t = 0; t < (terms == 3 ? 2 : 1); ++t)
                {
                    uint8_t *sb           = sb0 + t * Cfg::b_bytes;
                    const CUtensorMap *mb = t ? &tm.b_small : &tm.b;
                    if (!b_mn)
                    {
                        ptx::tma_load_2d_pair(sb, mb, bar, k0, nb0);
                    }
                    else if (b_mn & 2)
                    {
                        ptx::tma_load_3d_pair(sb, mb, bar, 0, k0, nb0 / 32);
                    }
                    else
                    {
#pragma unroll
                        for (int j = 0; j < BN / 64; ++j)
                            ptx::tma_load_2d_pair(sb + j * Cfg::mn_box, mb, bar, nb0 + 32 * j, k0);
                    }
                }
                }
                ++issued;
            }
            if (*abort_f && leader)
            {
                const int first = issued > stages ? issued - stages : 0;
                for (int kb = first; kb < issued; ++kb)
                    ptx::mbar_wait(&full_bar[kb % stages], (kb / stages) & 1, nullptr);
            }
        }
    }
    else if (warp == 1)
    {
        // ================================================================= MMA issuer (leader only)
        if (lane == 0 && leader)
        {
            const uint32_t idesc  = ptx::make_idesc_tf32(2 * kBM, BN, a_mn != 0, b_mn != 0);
            const uint32_t a_step = a_mn ? 1024u : 32u;
            const uint32_t b_step = b_mn ? 1024u : 32u;
            const uint32_t a_lbo  = a_mn ? Cfg::mn_box : 16u;
            const uint32_t b_lbo  = b_mn ? Cfg::mn_box : 16u;
            const uint32_t a_sbo  = a_mn ? 512u : 1024u;
            const uint32_t b_sbo  = b_mn ? 512u : 1024u;
            const uint32_t a_lay  = a_mn ? ptx::kLayoutSw128Base32 : ptx::kLayoutSw128;
            const uint32_t b_lay  = b_mn ? ptx::kLayoutSw128Base32 : ptx::kLayoutSw128;
            bool ok               = true;
            int kb                = 0;
            for (int c = 0; c < nchunks && ok; ++c)
            {
                const int buf         = c & 1;
                const uint32_t use    = static_cast<uint32_t>(c >> 1);
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
                        for (int kk = 0; kk < kBK / kUmmaK; ++kk)
                        {
                            const uint64_t da = ptx::make_smem_desc(sa + kk * a_step, a_lbo, a_sbo, a_lay);
                            const uint64_t db = ptx::make_smem_desc(sb + kk * b_step, b_lbo, b_sbo, b_lay);
                            if (terms == 3)
                            {
                                const uint64_t das = ptx::make_smem_desc(sas + kk * a_step, a_lbo, a_sbo, a_lay);
                                const uint64_t dbs = ptx::make_smem_desc(sbs + kk * b_step, b_lbo, b_sbo, b_lay);
                                ptx::mma_tf32_ss_pair(tmem_d, das, db, idesc, first ? 0u : 1u);
                                ptx::mma_tf32_ss_pair(tmem_d, da, dbs, idesc, 1);
                                ptx::mma_tf32_ss_pair(tmem_d, da, db, idesc, 1);
                            }
                            else
                            {
                                ptx::mma_tf32_ss_pair(tmem_d, da, db, idesc, first ? 0u : 1u);
                            }
                            first = false;
                    }
                    }
                    // the stage is free in BOTH CTAs once these MMAs have read it
                    ptx::mma_commit_pair_both(&empty_bar[s]);
                }
                if (ok)
                {
                    ptx::mma_commit_pair_both(&acc_full[buf]);
                }
            }
        }
    }
    else
    {
        // ================================================================= accumulate + epilogue (warps 2..9, both CTAs)
        const int e  = warp - 2;
        const int q  = warp & 3;
        const int h  = e >> 2;
        const int cw = h * Cfg::warp_cols;
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
                ptx::mbar_arrive_cluster(ptx::map_to_cta(ptx::smem_u32(&acc_empty[buf]), 0));
        }
        if (have)
            gemm_epilogue_store<256, Cfg::warp_cols>(p, acc, stg_all + e * 32 * kStgLd, m0, n0, cw, q, lane);
        ptx::tc_fence_before_sync();
    }

    // ---- teardown: nobody in the pair still uses TMEM or signals a barrier of the other CTA
    __syncthreads();
    ptx::cluster_sync();
    if (!skip && warp == 1)
    {
        __syncwarp();
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc_pair(tmem_base, Cfg::tmem_cols);
    }
    if (threadIdx.x == 0 && *abort_f && p.err != nullptr)
        atomicExch(p.err, 1);
}

// ---------------------------------------------------------------------------------------------------------------------
// Persistent 3xTF32 variant: as many CTA pairs as the GPU holds at once (74 on 148 SMs), each taking work units (tiles)
// off one list until it is empty.  Units are handed out in order by a counter in global memory: the leader's producer
// thread draws the next index and publishes it to every role of both CTAs through a two-slot mailbox (shared-memory
// slots + mbarriers, the peer's copy written through the cluster window).  Drawing instead of a fixed p, p + P, p + 2P
// assignment matters when the pairs do not all run at once -- another kernel (an NCCL all-reduce overlapping the
// backward pass) holds some SMs: pairs that start late then simply find fewer units left, instead of the whole GEMM
// waiting for a late pair to work through a fixed share.  Which pair computes a unit has no influence on its bits.
// What the kernel buys over one tile per pair:
//   * the epilogue of a tile (registers -> shared-memory slab -> global, with bias / ReLU / mask / column sums) runs
//     while the producer and the MMA thread are already on the next tile: the stage ring and the two TMEM accumulator
//     buffers simply keep rotating across tiles, so the MMA thread is ahead by two drains (128 of K) before it has to
//     wait for the epilogue warps, and set-up (barriers, TMEM allocation, first-load latency) is paid once per SM;
//   * the pairs start every round together, so a round's tiles stream the same K range at about the same time and
//     share their operand panels in L2 instead of drifting apart;
//   * a short last round is split along K: when the tiles left over after the full rounds would occupy at most half of
//     the pairs, each of them becomes TWO units (first and second half of K) on two pairs.  Both pairs park their
//     partial tile in scratch and take a ticket; whoever comes second adds the other's values to its own registers and
//     runs the epilogue.  Nobody waits for anybody, and a + b == b + a, so the result does not depend on who was second.
// Shared memory: three 64 KB stages, eight unpadded (XOR-swizzled) 4 KB transpose slabs beside the live ring, barriers.
struct PersistPlan
{
    int tiles_m, tiles_n;
    int full_units;   // whole tiles, one unit each: units [0, full_units)
    int split_tiles;  // tiles of the short last round, two units each: units [full_units, full_units + 2 * split_tiles)
    int num_kb;       // K-blocks of 32
    int kb_mid;       // first K-block of a split tile's second half
    int chunk_kb;     // K-blocks accumulated in TMEM between two drains
    // Stream-K mode (streamk != 0; for skinny outputs with at most half as many tiles as pairs): the tiles_m * tiles_n
    // * chunks_per_tile accumulator chunks of the whole problem are cut into one contiguous range per pair, pair p taking
    // chunks [p * C / P, (p + 1) * C / P): every pair gets the same amount of tensor work whatever the tile count.  A pair
    // then works on the tail of one tile, some whole tiles and the head of another; a tile cut by range boundaries is
    // finished by whichever of its contributors arrives last (tickets), adding the parked parts in part order.
    int streamk;
    int chunks_per_tile;  // ceil(num_kb / chunk_kb)
    int max_parts;        // slots per tile in `partial` (2 in the rounds mode)
    float *partial;   // [tile slots][max_parts][2 ranks][128 x 256] parked partial tiles
    unsigned *tickets;  // [tile slots][2 ranks], zero between launches (the last arriver resets its ticket)
    unsigned *counters;  // [0] next unit to hand out, [1] pairs that found the list empty; both zero between launches
                         // (the last pair to finish resets them); nullptr = fixed assignment p, p + P, ... (test hook)
};

constexpr int kPStages   = 3;
constexpr int kPSlab     = 32 * 32 * 4;  // one warp's transpose slab
constexpr int kMaxSkUnits = 32;          // units one pair's stream-K range may hold (the launcher checks)
constexpr int kPSmem     = 1024 + kPStages * PairCfg<256>::stage_bytes(3) + kEpiWarps * kPSlab + 256 + kMaxSkUnits * 6 * 4;

__device__ __forceinline__ void epilogue_warps_sync()
{
    asm volatile("bar.sync 1, %0;" ::"n"(32 * kEpiWarps) : "memory");
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_tc2_persistent_kernel(const __grid_constant__ TmapPack tm, const GemmParams p, const int a_mn, const int b_mn,
                           const PersistPlan plan)
{
    constexpr int BN = 256;
    using Cfg        = PairCfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *base = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int stage_bytes = Cfg::stage_bytes(3);
    uint8_t *tiles        = base;
    float *slabs          = reinterpret_cast<float *>(base + kPStages * stage_bytes);
    uint8_t *aux_base     = base + kPStages * stage_bytes + kEpiWarps * kPSlab;
    uint64_t *full_bar    = reinterpret_cast<uint64_t *>(aux_base);
    uint64_t *empty_bar   = full_bar + kPStages;
    uint64_t *acc_full    = empty_bar + kPStages;
    uint64_t *acc_empty   = acc_full + 2;
    uint32_t *tmem_slot   = reinterpret_cast<uint32_t *>(acc_empty + 2);
    volatile int *abort_f = reinterpret_cast<volatile int *>(tmem_slot + 1);
    int *early_out        = const_cast<int *>(abort_f) + 1;
    int *ticket_box       = early_out + 1;
    int *mail_slot        = ticket_box + 1;                                  // [2] unit index, -1 = list empty
    int *sk_count         = mail_slot + 2;                                   // units in sk_list
    int *sk_list          = reinterpret_cast<int *>(aux_base + 256);         // [kMaxSkUnits][6]: this pair's stream-K units
    uint64_t *mail_full   = reinterpret_cast<uint64_t *>(aux_base + 128);    // [2] per CTA: slot published
    uint64_t *mail_empty  = mail_full + 2;                                   // [2] leader's: all 18 readers have read

    const int warp      = threadIdx.x >> 5;
    const int lane      = threadIdx.x & 31;
    const uint32_t rank = ptx::cluster_ctarank();
    const bool leader   = rank == 0;
    const int pair      = blockIdx.x >> 1;
    const int n_pairs   = gridDim.x >> 1;
    const int n_units   = plan.full_units + 2 * plan.split_tiles;
    const bool drawn    = plan.counters != nullptr;

    if (threadIdx.x == 0)
    {
        *early_out = (leader && p.err != nullptr && *reinterpret_cast<volatile int *>(p.err) != 0) ? 1 : 0;
        *abort_f   = 0;
    }
    __syncthreads();
    ptx::cluster_sync();
    const bool skip = ptx::ld_shared_cluster_u32(ptx::map_to_cta(ptx::smem_u32(early_out), 0)) != 0;

    if (!skip)
    {
        if (warp == 0 && lane == 0)
        {
            ptx::prefetch_tmap(&tm.a);
            ptx::prefetch_tmap(&tm.b);
            ptx::prefetch_tmap(&tm.a_small);
            ptx::prefetch_tmap(&tm.b_small);
            for (int s = 0; s < kPStages; ++s)
            {
                ptx::mbar_init(&full_bar[s], 1);
                ptx::mbar_init(&empty_bar[s], 1);
            }
            for (int b = 0; b < 2; ++b)
            {
                ptx::mbar_init(&acc_full[b], 1);
                ptx::mbar_init(&acc_empty[b], 2 * kEpiWarps);
                ptx::mbar_init(&mail_full[b], 1);
                ptx::mbar_init(&mail_empty[b], 2 * (kEpiWarps + 1));  // per CTA: eight epilogue warps + MMA thread / producer
            }
            ptx::fence_mbar_init();
        }
        if (warp == 1)
        {
            ptx::tmem_alloc_pair(tmem_slot, Cfg::tmem_cols);
            ptx::tmem_relinquish_pair();
        }
        if (warp == 2 && lane == 0 && plan.streamk)
        {
            // Stream-K: the accumulator chunks of the whole problem, cut into one contiguous range per pair; this pair's
            // range as a list of units (tile, K-block range, part index / part count where a range boundary cuts the tile).
            const int pair_     = blockIdx.x >> 1;
            const int n_pairs_  = gridDim.x >> 1;
            const int nch       = plan.chunks_per_tile;
            const long long tot = static_cast<long long>(plan.tiles_m) * plan.tiles_n * nch;
            auto begin_of = [&](int pr) -> long long { return tot * pr / n_pairs_; };
            auto owner_of = [&](long long chunk) -> int {  // the pair whose range holds `chunk`
                int pr = static_cast<int>(chunk * n_pairs_ / tot);
                while (pr + 1 < n_pairs_ && begin_of(pr + 1) <= chunk)
                    ++pr;
                while (pr > 0 && begin_of(pr) > chunk)
                    --pr;
                return pr;
            };
            long long c = begin_of(pair_);
            const long long c_end = begin_of(pair_ + 1);
            int n = 0;
            while (c < c_end && n < kMaxSkUnits)
            {
                const int tile       = static_cast<int>(c / nch);
                const int ch_lo      = static_cast<int>(c - static_cast<long long>(tile) * nch);
                const long long left = c_end - c;
                const int ch_hi      = left >= nch - ch_lo ? nch : ch_lo + static_cast<int>(left);
                int part = -1, n_parts = 1;
                if (ch_lo != 0 || ch_hi != nch)
                {
                    const long long t0 = static_cast<long long>(tile) * nch;
                    const int first    = owner_of(t0), last = owner_of(t0 + nch - 1);
                    part               = pair_ - first;
                    n_parts            = last - first + 1;
                }
                int *e = sk_list + 6 * n++;
                e[0] = tile, e[1] = ch_lo * plan.chunk_kb, e[2] = min(plan.num_kb, ch_hi * plan.chunk_kb);
                e[3] = part, e[4] = n_parts, e[5] = tile;
                c += ch_hi - ch_lo;
            }
            *sk_count = n;
        }
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::cluster_sync();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = skip ? 0u : *tmem_slot;

    // ---- which unit is this pair's i-th?  Fixed assignment: pair + i * n_pairs.  Drawn: the leader's producer thread
    //      takes the next index off the global counter and puts it into mailbox slot i & 1 of BOTH CTAs (its peer's through
    //      the cluster window, released by the arrive that follows); every other role -- the peer's producer, the MMA
    //      thread, the sixteen epilogue warps -- waits for the slot, reads it and tells the leader it has (mail_empty).
    //      -1 ends the walk.  All waits are bounded like every other wait of the kernel.
    auto draw_and_publish = [&](uint32_t i) -> int {  // leader producer thread only
        if (!drawn)
        {
            const int u = pair + static_cast<int>(i) * n_pairs;
            return u < n_units ? u : -1;
        }
        const int slot = i & 1;
        if (!ptx::mbar_wait(&mail_empty[slot], ((i >> 1) & 1) ^ 1, abort_f))
            return -2;
        const unsigned got = atomicAdd(plan.counters, 1u);
        const int u        = got < static_cast<unsigned>(n_units) ? static_cast<int>(got) : -1;
        if (u < 0 && atomicAdd(plan.counters + 1, 1u) == static_cast<unsigned>(n_pairs - 1))
        {
            // every pair has now drawn past the end: nobody draws again in this launch; leave both counters at zero
            plan.counters[0] = 0;
            plan.counters[1] = 0;
        }
        mail_slot[slot] = u;
        ptx::st_shared_cluster_u32(ptx::map_to_cta(ptx::smem_u32(&mail_slot[slot]), 1), static_cast<uint32_t>(u));
        ptx::mbar_arrive_cluster(ptx::map_to_cta(ptx::smem_u32(&mail_full[slot]), 0));
        ptx::mbar_arrive_cluster(ptx::map_to_cta(ptx::smem_u32(&mail_full[slot]), 1));
        return u;
    };
    auto read_mail = [&](uint32_t i) -> int {  // one thread of every other role (a whole warp may call it: lane 0 acts)
        if (!drawn)
        {
            const int u = pair + static_cast<int>(i) * n_pairs;
            return u < n_units ? u : -1;
        }
        const int slot = i & 1;
        if (!ptx::mbar_wait_cluster(&mail_full[slot], (i >> 1) & 1, abort_f))
            return -2;
        const int u = *reinterpret_cast<volatile int *>(&mail_slot[slot]);
        ptx::mbar_arrive_cluster_relaxed(ptx::map_to_cta(ptx::smem_u32(&mail_empty[slot]), 0), static_cast<uint32_t>(u));
        return u;
    };

    // ---- a unit of work: a tile and a K-block range of it; `part` >= 0 marks a partial tile (part index in K order,
    //      n_parts contributors, tile_slot = where its parts are parked)
    struct Unit
    {
        int tile, kb0, kb1, part, n_parts, tile_slot;
    };
    // rounds mode: unit index -> unit
    auto unit_of_index = [&](int u) -> Unit {
        if (u < plan.full_units)
            return Unit{u, 0, plan.num_kb, -1, 1, 0};
        const int v = u - plan.full_units, half = v & 1;
        return Unit{plan.full_units + (v >> 1), half ? plan.kb_mid : 0, half ? plan.num_kb : plan.kb_mid, half, 2, v >> 1};
    };
    // next unit of this role.  Rounds mode: fetch(i) obtains the i-th unit index of this pair (draw / read the mailbox /
    // compute it).  Stream-K mode: the i-th entry of the list one thread made from this pair's chunk range during set-up
    // (the 64-bit range arithmetic stays out of the roles' registers).  Returns false when the walk is over (or a wait
    // gave up).
    struct Walk
    {
        uint32_t i = 0;
    };
    auto walk_init = [&](Walk &wk) { wk.i = 0; };
    // The same walk in two steps for the epilogue warps, which hold 128 accumulator registers while a unit is in flight:
    // a one-register token first, the unit's fields from it where they are needed (before and again after the drains).
    auto walk_token = [&](Walk &wk, auto &&fetch) -> int {
        if (plan.streamk)
            return static_cast<int>(wk.i) < *reinterpret_cast<volatile int *>(sk_count) ? static_cast<int>(wk.i++) : -1;
        return fetch(wk.i++);
    };
    auto unit_from = [&](int token) -> Unit {
        if (plan.streamk)
        {
            const volatile int *e = sk_list + 6 * token;
            return Unit{e[0], e[1], e[2], e[3], e[4], e[5]};
        }
        return unit_of_index(token);
    };
    auto walk_next = [&](Walk &wk, auto &&fetch, Unit &out) -> bool {
        if (plan.streamk)
        {
            if (static_cast<int>(wk.i) >= *reinterpret_cast<volatile int *>(sk_count))
                return false;
            const int *e = sk_list + 6 * wk.i++;
            out          = Unit{e[0], e[1], e[2], e[3], e[4], e[5]};
            return true;
        }
        const int u = fetch(wk.i++);
        if (u < 0)
            return false;
        out = unit_of_index(u);
        return true;
    };

    auto tile_origin = [&](int tile, int &tile_m, int &tile_n) {
        const int per_group = kGroupM * plan.tiles_n;
        const int g         = tile / per_group;
        const int first_m   = g * kGroupM;
        const int gsz       = min(plan.tiles_m - first_m, kGroupM);
        const int local     = tile - g * per_group;
        tile_m              = first_m + local % gsz;
        tile_n              = local / gsz;
    };

    if (skip)
    {
        // nothing
    }
    else if (warp == 0)
    {
        // ================================================================= TMA producer (both CTAs)
        if (lane == 0)
        {
            uint32_t gk = 0;  // K-blocks issued so far: the ring position carries over from tile to tile
            bool ok     = true;
            Walk wk;
            walk_init(wk);
            Unit un;
            while (ok && walk_next(wk, [&](uint32_t i) { return leader ? draw_and_publish(i) : read_mail(i); }, un))
            {
                int tile_m, tile_n;
                tile_origin(un.tile, tile_m, tile_n);
                const int kb0 = un.kb0, kb1 = un.kb1;
                const int m0  = tile_m * 2 * kBM + static_cast<int>(rank) * kBM;
                const int nb0 = tile_n * BN + static_cast<int>(rank) * (BN / 2);
                for (int kb = kb0; kb < kb1; ++kb, ++gk)
                {
                    const int s       = gk % kPStages;
                    const uint32_t ph = (gk / kPStages) & 1;
                    if (!ptx::mbar_wait(&empty_bar[s], ph ^ 1, abort_f))
                    {
                        ok = false;
                        break;
                    }
                    if (leader)
                        ptx::mbar_arrive_expect_tx(&full_bar[s], 2 * stage_bytes);
                    const uint32_t bar = ptx::map_to_cta(ptx::smem_u32(&full_bar[s]), 0);
                    uint8_t *st  = tiles + s * stage_bytes;
                    const int k0 = kb * kBK;
#pragma unroll
                    for (int t = 0; t < 2; ++t)
                    {
                        uint8_t *sa           = st + t * Cfg::a_bytes;
                        const CUtensorMap *ma = t ? &tm.a_small : &tm.a;
                        if (!a_mn)
                            ptx::tma_load_2d_pair(sa, ma, bar, k0, m0);
                        else if (a_mn & 2)
                            ptx::tma_load_3d_pair(sa, ma, bar, 0, k0, m0 / 32);
                        else
                            for (int j = 0; j < kBM / 32; ++j)
                                ptx::tma_load_2d_pair(sa + j * Cfg::mn_box, ma, bar, m0 + 32 * j, k0);
                    }
                    uint8_t *sb0 = st + 2 * Cfg::a_bytes;
#pragma unroll
                    for (int t = 0; t < 2; ++t)
                    {
                        uint8_t *sb           = sb0 + t * Cfg::b_bytes;
                        const CUtensorMap *mb = t ? &tm.b_small : &tm.b;
                        if (!b_mn)
                            ptx::tma_load_2d_pair(sb, mb, bar, k0, nb0);
                        else if (b_mn & 2)
                            ptx::tma_load_3d_pair(sb, mb, bar, 0, k0, nb0 / 32);
                        else
                            for (int j = 0; j < BN / 64; ++j)
                                ptx::tma_load_2d_pair(sb + j * Cfg::mn_box, mb, bar, nb0 + 32 * j, k0);
                    }
                }
            }
            if (*abort_f && leader)
            {
                // let the copies still in flight land before the CTA goes away
                const uint32_t first = gk > kPStages ? gk - kPStages : 0;
                for (uint32_t k = first; k < gk; ++k)
                    ptx::mbar_wait(&full_bar[k % kPStages], (k / kPStages) & 1, nullptr);
            }
        }
    }
    else if (warp == 1)
    {
        // ================================================================= MMA issuer (leader only)
        if (lane == 0 && leader)
        {
            const uint32_t idesc  = ptx::make_idesc_tf32(2 * kBM, BN, a_mn != 0, b_mn != 0);
            const uint32_t a_step = a_mn ? 1024u : 32u;
            const uint32_t b_step = b_mn ? 1024u : 32u;
            const uint32_t a_lbo  = a_mn ? Cfg::mn_box : 16u;
            const uint32_t b_lbo  = b_mn ? Cfg::mn_box : 16u;
            const uint32_t a_sbo  = a_mn ? 512u : 1024u;
            const uint32_t b_sbo  = b_mn ? 512u : 1024u;
            const uint32_t a_lay  = a_mn ? ptx::kLayoutSw128Base32 : ptx::kLayoutSw128;
            const uint32_t b_lay  = b_mn ? ptx::kLayoutSw128Base32 : ptx::kLayoutSw128;
            uint32_t gk = 0, gc = 0;  // K-blocks consumed and accumulator chunks started so far, over all tiles
            bool ok     = true;
            Walk wk;
            walk_init(wk);
            Unit un;
            while (ok && walk_next(wk, read_mail, un))
            {
                const int kb0 = un.kb0, kb1 = un.kb1;
                for (int kb = kb0; kb < kb1 && ok; ++gc)
                {
                    const int buf         = gc & 1;
                    const uint32_t use    = gc >> 1;
                    const uint32_t tmem_d = tmem_base + buf * BN;
                    if (!ptx::mbar_wait(&acc_empty[buf], (use & 1) ^ 1, abort_f))
                    {
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after_sync();
                    const int kb_end = min(kb + plan.chunk_kb, kb1);
                    for (bool first = true; kb < kb_end; ++kb, ++gk)
                    {
                        const int s       = gk % kPStages;
                        const uint32_t ph = (gk / kPStages) & 1;
                        if (!ptx::mbar_wait(&full_bar[s], ph, abort_f))
                        {
                            ok = false;
                            break;
                        }
                        ptx::tc_fence_after_sync();
                        const uint32_t sa  = ptx::smem_u32(tiles + s * stage_bytes);
                        const uint32_t sas = sa + Cfg::a_bytes;
                        const uint32_t sb  = sa + 2 * Cfg::a_bytes;
                        const uint32_t sbs = sb + Cfg::b_bytes;
#pragma unroll
                        for (int kk = 0; kk < kBK / kUmmaK; ++kk)
                        {
                            const uint64_t da  = ptx::make_smem_desc(sa + kk * a_step, a_lbo, a_sbo, a_lay);
                            const uint64_t db  = ptx::make_smem_desc(sb + kk * b_step, b_lbo, b_sbo, b_lay);
                            const uint64_t das = ptx::make_smem_desc(sas + kk * a_step, a_lbo, a_sbo, a_lay);
                            const uint64_t dbs = ptx::make_smem_desc(sbs + kk * b_step, b_lbo, b_sbo, b_lay);
                            ptx::mma_tf32_ss_pair(tmem_d, das, db, idesc, first ? 0u : 1u);
                            ptx::mma_tf32_ss_pair(tmem_d, da, dbs, idesc, 1);
                            ptx::mma_tf32_ss_pair(tmem_d, da, db, idesc, 1);
                            first = false;
                        }
                        ptx::mma_commit_pair_both(&empty_bar[s]);
                    }
                    if (ok)
                        ptx::mma_commit_pair_both(&acc_full[buf]);
                }
            }
        }
    }
    else
    {
        // ================================================================= accumulate + epilogue (warps 2..9, both CTAs)
        const int e  = warp - 2;
        const int q  = warp & 3;
        const int h  = e >> 2;
        const int cw = h * Cfg::warp_cols;
        float *slab  = slabs + e * (kPSlab / 4);
        const bool direct = epilogue_direct_ok(p);  // rows of D from registers with 256-bit stores, no transpose slab
        float acc[Cfg::warp_cols];
        uint32_t gc = 0;
        bool have   = true;
        Walk wk;
        walk_init(wk);
        // (every lane walks: in the drawn mode lane 0 reads the mailbox and the index is broadcast)
        auto warp_fetch = [&](uint32_t i) -> int {
            int u = 0;
            if (lane == 0)
                u = read_mail(i);
            return __shfl_sync(0xffffffffu, u, 0);
        };
        int token;
        while (have && (token = walk_token(wk, warp_fetch)) >= 0)
        {
            int nchunks;
            {
                const Unit first = unit_from(token);
                nchunks          = (first.kb1 - first.kb0 + plan.chunk_kb - 1) / plan.chunk_kb;
            }
            for (int c = 0; c < nchunks; ++c, ++gc)
            {
                const int buf      = gc & 1;
                const uint32_t use = gc >> 1;
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
                // relaxed: the buffer's TMEM reads are complete (wait::ld) and fenced; a release at cluster scope would also
                // wait for the global stores of the tile this warp has just written, behind every tile
                if (lane == 0)
                    ptx::mbar_arrive_cluster_relaxed(ptx::map_to_cta(ptx::smem_u32(&acc_empty[buf]), 0));
            }
            if (!have)
                break;
            const Unit un = unit_from(token);
            int tile_m, tile_n;
            tile_origin(un.tile, tile_m, tile_n);
            const int m0 = tile_m * 2 * kBM + static_cast<int>(rank) * kBM;
            const int n0 = tile_n * BN;
            bool store   = true;
            if (un.part >= 0)
            {
                // part of a tile: park it, take a ticket; whoever holds the LAST ticket adds all parts in part order (a
                // fixed order, whoever it is -- its own part is read back from its slot like the others) and stores
                // parts of this tile, this CTA's half: slot (tile_slot * max_parts + part) * 2 + rank, kBM * BN floats each
                float4 *const parts0 = reinterpret_cast<float4 *>(plan.partial) +
                                       (static_cast<size_t>(un.tile_slot) * plan.max_parts * 2 + rank) * (kBM * BN / 4) +
                                       (e * 32) * 32 + lane;
                auto slot_ptr = [&](int part) { return parts0 + static_cast<size_t>(part) * (2 * kBM * BN / 4); };
                float4 *mine = slot_ptr(un.part);
#pragma unroll
                for (int i = 0; i < Cfg::warp_cols / 4; ++i)
                    mine[i * 32] = make_float4(acc[4 * i], acc[4 * i + 1], acc[4 * i + 2], acc[4 * i + 3]);
                __threadfence();  // this thread's part of the partial tile is visible device-wide before the ticket is taken
                epilogue_warps_sync();
                unsigned *ticket = plan.tickets + un.tile_slot * 2 + rank;
                if (warp == 2 && lane == 0)
                {
                    __threadfence();
                    *ticket_box = static_cast<int>(atomicAdd(ticket, 1u));
                }
                epilogue_warps_sync();
                store = *ticket_box == un.n_parts - 1;
                if (store)
                {
                    __threadfence();
                    {
                        const float4 *src = slot_ptr(0);
#pragma unroll
                        for (int i = 0; i < Cfg::warp_cols / 4; ++i)
                        {
                            const float4 o = __ldcg(src + i * 32);
                            acc[4 * i] = o.x, acc[4 * i + 1] = o.y, acc[4 * i + 2] = o.z, acc[4 * i + 3] = o.w;
                        }
                    }
#pragma unroll 1
                    for (int part = 1; part < un.n_parts; ++part)
                    {
                        const float4 *src = slot_ptr(part);
#pragma unroll
                        for (int i = 0; i < Cfg::warp_cols / 4; ++i)
                        {
                            const float4 o = __ldcg(src + i * 32);
                            acc[4 * i] += o.x, acc[4 * i + 1] += o.y, acc[4 * i + 2] += o.z, acc[4 * i + 3] += o.w;
                        }
                    }
                }
                epilogue_warps_sync();  // everybody has read the ticket before the next unit may overwrite the box
                if (store && warp == 2 && lane == 0)
                    *ticket = 0;  // ready for the next launch
            }
            if (store)
            {
                if (direct)
                    gemm_epilogue_direct<Cfg::warp_cols>(p, acc, m0, n0, cw, q, lane);
                else
                    gemm_epilogue_store<256, Cfg::warp_cols, true>(p, acc, slab, m0, n0, cw, q, lane);
            }
        }
        ptx::tc_fence_before_sync();
    }

    // ---- teardown: nobody in the pair still uses TMEM or signals a barrier of the other CTA
    __syncthreads();
    ptx::cluster_sync();
    if (!skip && warp == 1)
    {
        __syncwarp();
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc_pair(tmem_base, Cfg::tmem_cols);
    }
    if (threadIdx.x == 0 && *abort_f && p.err != nullptr)
        atomicExch(p.err, 1);
}

// ---------------------------------------------------------------------------------------------------------------------
// Plain-TF32 variant with a 256 x 512 tile per pair.  Plain TF32 never drains the accumulator mid-way, so the second
// TMEM buffer of the kernel above is free to hold 256 more columns: each CTA then loads one 128-row A tile and TWO
// 128-row blocks of B per K-slab (48 KB for 2 x 128 x 256 x 32 products instead of 32 KB for half of that), i.e. 0.75 of
// the operand bytes per product.  That matters because plain TF32 on this kernel is bound by what the L2 -> SM fabric
// delivers (about 8-10 TB/s over all SMs), not by the tensor pipe.  Per K-slab the leader issues 4 K-steps x 2 MMAs
// (N = 256 each, columns 0..255 and 256..511 of the accumulator).  Four 48 KB stages; the epilogue streams the
// accumulator out of TMEM 32 columns at a time.
constexpr int kWideBN     = 512;
constexpr int kWideBBlock = 128 * kBK * 4;               // one 128-row block of B
constexpr int kWideStage  = kBM * kBK * 4 + 2 * kWideBBlock;  // 48 KB
constexpr int kWideStages = 4;
constexpr int kWideSmem   = 1024 + kAuxBytes + kWideStages * kWideStage;

__global__ void __launch_bounds__(kThreads, 1)
gemm_tc2_wide_kernel(const __grid_constant__ TmapPack tm, const GemmParams p, const int a_mn, const int b_mn)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t *base = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *tiles        = base;
    float *stg_all        = reinterpret_cast<float *>(base);
    uint8_t *aux_base     = base + kWideStages * kWideStage;
    uint64_t *full_bar    = reinterpret_cast<uint64_t *>(aux_base);
    uint64_t *empty_bar   = full_bar + kMaxStages;
    uint64_t *acc_full    = empty_bar + kMaxStages;
    uint32_t *tmem_slot   = reinterpret_cast<uint32_t *>(acc_full + 4);
    volatile int *abort_f = reinterpret_cast<volatile int *>(tmem_slot + 1);
    int *early_out        = const_cast<int *>(abort_f) + 1;

    const int warp      = threadIdx.x >> 5;
    const int lane      = threadIdx.x & 31;
    const uint32_t rank = ptx::cluster_ctarank();
    const bool leader   = rank == 0;

    if (threadIdx.x == 0)
    {
        *early_out = (leader && p.err != nullptr && *reinterpret_cast<volatile int *>(p.err) != 0) ? 1 : 0;
        *abort_f   = 0;
    }
    __syncthreads();
    ptx::cluster_sync();
    const bool skip = ptx::ld_shared_cluster_u32(ptx::map_to_cta(ptx::smem_u32(early_out), 0)) != 0;

    const int tiles_m = (p.M + 2 * kBM - 1) / (2 * kBM);
    const int tiles_n = (p.N + kWideBN - 1) / kWideBN;
    int tile_m, tile_n;
    {
        const int pair      = blockIdx.x >> 1;
        const int per_group = kGroupM * tiles_n;
        const int g         = pair / per_group;
        const int first_m   = g * kGroupM;
        const int gsz       = min(tiles_m - first_m, kGroupM);
        const int local     = pair - g * per_group;
        tile_m              = first_m + local % gsz;
        tile_n              = local / gsz;
    }
    const int m0     = tile_m * 2 * kBM + static_cast<int>(rank) * kBM;
    const int n0     = tile_n * kWideBN;
    const int num_kb = (p.K + kBK - 1) / kBK;

    if (!skip)
    {
        if (warp == 0 && lane == 0)
        {
            ptx::prefetch_tmap(&tm.a);
            ptx::prefetch_tmap(&tm.b);
            for (int s = 0; s < kWideStages; ++s)
            {
                ptx::mbar_init(&full_bar[s], 1);
                ptx::mbar_init(&empty_bar[s], 1);
            }
            ptx::mbar_init(acc_full, 1);
            ptx::fence_mbar_init();
        }
        if (warp == 1)
        {
            ptx::tmem_alloc_pair(tmem_slot, 512);
            ptx::tmem_relinquish_pair();
        }
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::cluster_sync();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = skip ? 0u : *tmem_slot;

    if (skip)
    {
        // nothing
    }
    else if (warp == 0)
    {
        // ================================================================= TMA producer (both CTAs)
        if (lane == 0)
        {
            int issued = 0;
            for (int kb = 0; kb < num_kb; ++kb)
            {
                const int s       = kb % kWideStages;
                const uint32_t ph = (kb / kWideStages) & 1;
                if (!ptx::mbar_wait(&empty_bar[s], ph ^ 1, abort_f))
                    break;
                if (leader)
                    ptx::mbar_arrive_expect_tx(&full_bar[s], 2 * kWideStage);
                const uint32_t bar = ptx::map_to_cta(ptx::smem_u32(&full_bar[s]), 0);
                uint8_t *sa  = tiles + s * kWideStage;
                const int k0 = kb * kBK;
                if (!a_mn)
                    ptx::tma_load_2d_pair(sa, &tm.a, bar, k0, m0);
                else if (a_mn & 2)
                    ptx::tma_load_3d_pair(sa, &tm.a, bar, 0, k0, m0 / 32);
                else
                    for (int j = 0; j < kBM / 32; ++j)
                        ptx::tma_load_2d_pair(sa + j * 4096, &tm.a, bar, m0 + 32 * j, k0);
                for (int blk = 0; blk < 2; ++blk)
                {
                    // block blk of this CTA: rows n0 + 256 blk + 128 rank .. + 127 of B (its half of MMA number blk)
                    uint8_t *sb   = sa + kBM * kBK * 4 + blk * kWideBBlock;
                    const int nb0 = n0 + 256 * blk + 128 * static_cast<int>(rank);
                    if (!b_mn)
                        ptx::tma_load_2d_pair(sb, &tm.b, bar, k0, nb0);
                    else if (b_mn & 2)
                        ptx::tma_load_3d_pair(sb, &tm.b, bar, 0, k0, nb0 / 32);
                    else
                        for (int j = 0; j < 4; ++j)
                            ptx::tma_load_2d_pair(sb + j * 4096, &tm.b, bar, nb0 + 32 * j, k0);
                }
                ++issued;
            }
            if (*abort_f && leader)
            {
                const int first = issued > kWideStages ? issued - kWideStages : 0;
                for (int kb = first; kb < issued; ++kb)
                    ptx::mbar_wait(&full_bar[kb % kWideStages], (kb / kWideStages) & 1, nullptr);
            }
        }
    }
    else if (warp == 1)
    {
        // ================================================================= MMA issuer (leader only)
        if (lane == 0 && leader)
        {
            const uint32_t idesc  = ptx::make_idesc_tf32(2 * kBM, 256, a_mn != 0, b_mn != 0);
            const uint32_t a_step = a_mn ? 1024u : 32u;
            const uint32_t b_step = b_mn ? 1024u : 32u;
            const uint32_t a_lbo  = a_mn ? 4096u : 16u;
            const uint32_t b_lbo  = b_mn ? 4096u : 16u;
            const uint32_t a_sbo  = a_mn ? 512u : 1024u;
            const uint32_t b_sbo  = b_mn ? 512u : 1024u;
            const uint32_t a_lay  = a_mn ? ptx::kLayoutSw128Base32 : ptx::kLayoutSw128;
            const uint32_t b_lay  = b_mn ? ptx::kLayoutSw128Base32 : ptx::kLayoutSw128;
            bool ok               = true;
            for (int kb = 0; kb < num_kb; ++kb)
            {
                const int s       = kb % kWideStages;
                const uint32_t ph = (kb / kWideStages) & 1;
                if (!ptx::mbar_wait(&full_bar[s], ph, abort_f))
                {
                    ok = false;
                    break;
                }
                ptx::tc_fence_after_sync();
                const uint32_t sa = ptx::smem_u32(tiles + s * kWideStage);
                const uint32_t sb = sa + kBM * kBK * 4;
#pragma unroll
                for (int kk = 0; kk < kBK / kUmmaK; ++kk)
                {
                    const uint64_t da   = ptx::make_smem_desc(sa + kk * a_step, a_lbo, a_sbo, a_lay);
                    const uint64_t db0  = ptx::make_smem_desc(sb + kk * b_step, b_lbo, b_sbo, b_lay);
                    const uint64_t db1  = ptx::make_smem_desc(sb + kWideBBlock + kk * b_step, b_lbo, b_sbo, b_lay);
                    const uint32_t accf = (kb == 0 && kk == 0) ? 0u : 1u;
                    ptx::mma_tf32_ss_pair(tmem_base, da, db0, idesc, accf);
                    ptx::mma_tf32_ss_pair(tmem_base + 256, da, db1, idesc, accf);
                }
                ptx::mma_commit_pair_both(&empty_bar[s]);
            }
            if (ok)
                ptx::mma_commit_pair_both(acc_full);
        }
    }
    else
    {
        // ================================================================= epilogue (warps 2..9, both CTAs)
        const int e  = warp - 2;
        const int q  = warp & 3;
        const int h  = e >> 2;
        const int cw = h * 256;  // this warp streams columns cw .. cw + 255 of the 512-wide tile
        const bool have = __all_sync(0xffffffffu, ptx::mbar_wait(acc_full, 0, abort_f));
        if (have)
        {
            ptx::tc_fence_after_sync();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(32 * q) << 16) + cw;
            for (int j = 0; j < 8; ++j)
            {
                if (n0 + cw + 32 * j >= p.N)
                    break;
                uint32_t r[32];
                float acc[32];
                ptx::tmem_ld_32x32(taddr + 32 * j, r);
                ptx::tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    acc[i] = __uint_as_float(r[i]);
                // the operand ring is dead (acc_full fired): its first bytes serve as the per-warp transpose slabs
                gemm_epilogue_store<256, 32>(p, acc, stg_all + e * 32 * kStgLd, m0, n0, cw + 32 * j, q, lane);
            }
        }
        ptx::tc_fence_before_sync();
    }

    __syncthreads();
    ptx::cluster_sync();
    if (!skip && warp == 1)
    {
        __syncwarp();
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc_pair(tmem_base, 512);
    }
    if (threadIdx.x == 0 && *abort_f && p.err != nullptr)
        atomicExch(p.err, 1);
}

}  // namespace

// Test hook: 0 = use the pair kernel where it pays (automatic), 1 = never, 2 = whenever the shape allows it,
// 3 = separate 2-D copies for MN-major operands, 4 = never the 256 x 512 plain-TF32 tile, 5 = like 2 and the 256 x 512
// tile for every plain-TF32 problem, 6 = never the persistent kernel, 7 = like 2 and the persistent kernel for every
// 3xTF32 problem.
int g_pair_mode = 0;
// Test hook: CTA pairs the persistent kernel uses (0 = as many as the GPU holds at once).
int g_persist_pairs = 0;
// Test hook: 0 = stream-K where it pays, 1 = for every problem the persistent kernel takes, -1 = never.
int g_stream_k = 0;
extern int g_slabs;

namespace
{
// Scratch of the persistent kernel's split last round: parked partial tiles and their tickets.  Grown on demand (the
// device is drained first), never shrunk; tickets are zero between launches.
float *g_part           = nullptr;
size_t g_part_floats    = 0;
unsigned *g_tickets     = nullptr;
size_t g_ticket_count   = 0;

// Unit counters of the persistent kernel: a ring of (next unit, finished pairs) slots, one slot per launch in turn, so
// that launches in flight on different streams never share one.  A launch leaves its slot at zero.
constexpr int kCounterSlots = 32;
unsigned *g_counters        = nullptr;
unsigned g_counter_seq      = 0;

int unit_counters(unsigned **out)
{
    if (!g_counters)
    {
        if (cudaMalloc(&g_counters, kCounterSlots * 2 * sizeof(unsigned)) != cudaSuccess ||
            cudaMemset(g_counters, 0, kCounterSlots * 2 * sizeof(unsigned)) != cudaSuccess)
        {
            g_counters = nullptr;
            set_last_error("gemm: cannot allocate the unit counters of the persistent kernel");
            return kCudaError;
        }
    }
    *out = g_counters + 2 * (g_counter_seq++ % kCounterSlots);
    return kOk;
}

int tail_split_scratch(size_t floats, size_t tickets)
{
    if (floats <= g_part_floats && tickets <= g_ticket_count)
        return kOk;
    if (cudaDeviceSynchronize() != cudaSuccess)
        return kCudaError;
    cudaFree(g_part);
    cudaFree(g_tickets);
    g_part = nullptr, g_tickets = nullptr, g_part_floats = 0, g_ticket_count = 0;
    tickets = tickets < 256 ? 256 : tickets;
    if (cudaMalloc(&g_part, floats * 4) != cudaSuccess || cudaMalloc(&g_tickets, tickets * 4) != cudaSuccess ||
        cudaMemset(g_tickets, 0, tickets * 4) != cudaSuccess)
    {
        set_last_error("gemm: cannot allocate %zu bytes of scratch for the split last round", floats * 4 + tickets * 4);
        return kCudaError;
    }
    g_part_floats = floats, g_ticket_count = tickets;
    bump_scratch_generation();
    return kOk;
}

// CTA pairs of the persistent kernel the device holds at once (74 on a full B200), asked of the driver once per device.
int resident_pairs()
{
    static int cached[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    dev &= 63;
    if (cached[dev] == 0)
    {
        cudaFuncSetAttribute(gemm_tc2_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPSmem);
        cudaDeviceProp prop;
        int sms = cudaGetDeviceProperties(&prop, dev) == cudaSuccess ? prop.multiProcessorCount : 148;
        cudaLaunchConfig_t cfg;
        std::memset(&cfg, 0, sizeof(cfg));
        cfg.gridDim          = dim3(static_cast<unsigned>(sms & ~1), 1, 1);
        cfg.blockDim         = dim3(kThreads, 1, 1);
        cfg.dynamicSmemBytes = kPSmem;
        cudaLaunchAttribute attr[1];
        attr[0].id               = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs                = attr;
        cfg.numAttrs             = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, gemm_tc2_persistent_kernel, &cfg) != cudaSuccess || n <= 0)
        {
            cudaGetLastError();
            n = -1;  // unknown: the persistent kernel stays off on this device
        }
        cached[dev] = n;
    }
    return cached[dev];
}
}  // namespace

// True when gemm_tc_launch should hand this problem to the pair kernel: whenever there is at least one pair per two SMs.
// Measured on B200 at 8192^3 with the kernels alternated inside one run (the GPU sits at its power cap during long
// runs, so numbers taken minutes apart differ by up to 8 %), TFLOP/s, 1-CTA -> pairs:
//   3xTF32: K-major x K-major 203 -> 225, with an MN-major operand 181 -> 225 (the 1-CTA kernel saturates its SM's
//           shared-memory bandwidth: 240 KB per K-block against 160 KB per CTA of a pair);
//   TF32 with two K-slabs per stage: K-major x K-major 533 -> 652, MN-major B 443 -> 583, both MN-major 399 -> 506
//           (with one slab per stage the pair kernel was the slower one for K-major operands: 473).
// After a kernel gave up on a bounded wait the persistent kernel may have left its unit counters and tickets in the
// middle of a launch: put them back to zero (called by odl_device_status when it reports the time-out).
int gemm_pair_recover(cudaStream_t stream)
{
    if (g_counters && cudaMemsetAsync(g_counters, 0, kCounterSlots * 2 * sizeof(unsigned), stream) != cudaSuccess)
        return kCudaError;
    if (g_tickets && cudaMemsetAsync(g_tickets, 0, g_ticket_count * sizeof(unsigned), stream) != cudaSuccess)
        return kCudaError;
    return kOk;
}

bool gemm_pair_eligible(const GemmParams &p, int bn, int a_mn, int b_mn, int terms)
{
    (void)a_mn, (void)b_mn;
    if (g_pair_mode == 1 || bn != 256 || p.M <= kBM || (p.flags & (kEpiNCHW | kEpiSplitK)))
        return false;
    if (g_pair_mode == 2 || g_pair_mode == 5 || g_pair_mode == 7)
        return true;
    const int64_t pairs = static_cast<int64_t>((p.M + 255) / 256) * ((p.N + 255) / 256);
    if (pairs >= 74)
        return true;
    // fewer tiles than pairs: the persistent kernel in stream-K mode still fills the GPU when the reduction is long
    // enough to cut (3xTF32 only; at least eight accumulator chunks = 512 of K per pair)
    const int64_t chunks = pairs * ((p.K + 63) / 64);
    return terms == 3 && g_pair_mode != 6 && g_stream_k >= 0 && pairs >= 16 && chunks >= 8 * 74;
}

int gemm_pair_launch(const float *A, const float *A_small, int64_t lda, int a_mn, const float *B, const float *B_small,
                     int64_t ldb, int b_mn, const GemmParams &p, int terms, cudaStream_t stream)
{
    constexpr int BN = 256;
    using Cfg        = PairCfg<BN>;
    TmapPack tm;
    std::memset(&tm, 0, sizeof(tm));
    int rc;
    // MN-major operands whose extent is a multiple of 32: one 3-D copy per operand and K-slab instead of one 2-D copy
    // per 32 x 32 box (the producer thread otherwise issues 16 copies per stage, which bounds plain TF32)
    CUtensorMap probe;
    if (a_mn && make_tmap_mn3d(&probe, A, p.K, p.M, lda, kBK, kBM / 32, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B) == kOk)
        a_mn |= 2;
    if (b_mn && make_tmap_mn3d(&probe, B, p.K, p.N, ldb, kBK, BN / 64, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B) == kOk)
        b_mn |= 2;
    if (g_pair_mode == 3)
        a_mn &= 1, b_mn &= 1;  // test hook: separate 2-D copies
    auto mk = [&](CUtensorMap *m, const float *ptr, int64_t ld, int mn, int64_t extent_mn, int box_rows_kmajor) {
        if (mn & 2)
            return make_tmap_mn3d(m, ptr, p.K, extent_mn, ld, kBK, box_rows_kmajor / 32, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
        return mn ? make_tmap(m, ptr, p.K, extent_mn, ld, 32, kBK, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B)
                  : make_tmap(m, ptr, extent_mn, p.K, ld, kBK, box_rows_kmajor, CU_TENSOR_MAP_SWIZZLE_128B);
    };
    if ((rc = mk(&tm.a, A, lda, a_mn, p.M, kBM)))
        return rc;
    if ((rc = mk(&tm.b, B, ldb, b_mn, p.N, BN / 2)))
        return rc;
    if (terms == 3)
    {
        if ((rc = mk(&tm.a_small, A_small, lda, a_mn, p.M, kBM)))
            return rc;
        if ((rc = mk(&tm.b_small, B_small, ldb, b_mn, p.N, BN / 2)))
            return rc;
    }
    // plain TF32, plain drains, enough 256 x 512 tiles for every pair of SMs: the wide tile (fewer operand bytes per
    // product); g_slabs / g_chunk_kb (test hooks of the narrow kernel) turn it off
    const int64_t wide_pairs = static_cast<int64_t>((p.M + 255) / 256) * ((p.N + kWideBN - 1) / kWideBN);
    if (terms == 1 && g_pair_mode != 4 && g_slabs == 0 && g_chunk_kb == 0 &&
        (g_pair_mode == 5 || (wide_pairs >= 74 && (p.N % kWideBN == 0 || p.N >= 8 * kWideBN) && p.K >= 4 * kBK)))
    {
        static bool wide_attr[64] = {};
        int dev = 0;
        cudaGetDevice(&dev);
        dev &= 63;
        if (!wide_attr[dev])
        {
            cudaError_t e = cudaFuncSetAttribute(gemm_tc2_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kWideSmem);
            if (e != cudaSuccess)
            {
                set_last_error("cudaFuncSetAttribute(wide pair kernel, smem=%d) failed: %s", kWideSmem, cudaGetErrorString(e));
                return kCudaError;
            }
            wide_attr[dev] = true;
        }
        cudaLaunchConfig_t cfg;
        std::memset(&cfg, 0, sizeof(cfg));
        cfg.gridDim          = dim3(static_cast<unsigned>(2 * wide_pairs), 1, 1);
        cfg.blockDim         = dim3(kThreads, 1, 1);
        cfg.dynamicSmemBytes = kWideSmem;
        cfg.stream           = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id               = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs                = attr;
        cfg.numAttrs             = 1;
        cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc2_wide_kernel, tm, p, a_mn, b_mn);
        ++g_launch_count;
        if (e != cudaSuccess)
        {
            set_last_error("gemm_tc2_wide_kernel launch failed: %s", cudaGetErrorString(e));
            return kCudaError;
        }
        return kOk;
    }
    // 3xTF32: the persistent kernel (epilogue overlapped with the next tile's main loop, short last round split along K).
    // g_pair_mode 2 and 6 = never (one tile per pair launch instead).
    if (terms == 3 && g_pair_mode != 6 && g_pair_mode != 3 && g_pair_mode != 2)
    {
        const int tiles_m = (p.M + 2 * kBM - 1) / (2 * kBM), tiles_n = (p.N + BN - 1) / BN;
        const int T       = tiles_m * tiles_n;
        int P             = resident_pairs();
        const int want_p  = g_persist_pairs < 0 ? -g_persist_pairs : g_persist_pairs;
        if (want_p > 0 && P > 0)
            P = want_p < P ? want_p : P;
        const int num_kb    = (p.K + kBK - 1) / kBK;
        int chunk_kb        = g_chunk_kb > 0 ? g_chunk_kb : 64 / kBK;
        if (chunk_kb > num_kb)
            chunk_kb = num_kb;
        const int nch       = (num_kb + chunk_kb - 1) / chunk_kb;
        // At most half as many tiles as pairs (a skinny output with a long reduction: 256 x 8192 x 8192 has 32 tiles):
        // whole tiles would leave most pairs idle, so the K ranges are cut evenly over all pairs (stream-K).  Measured on
        // B200 (TFLOP/s, whole tiles -> stream-K): 256 x 8192 x 8192 158-177 -> 174-187.  With more tiles it LOSES --
        // 2048^3 (64 tiles) 175 -> 158, 8192 x 1024 x 8192 (128 tiles) 223 -> 206, 3072^3 204 -> 179 -- because pairs that
        // share an operand panel then sit at different K offsets and stop sharing it in L2, which rounds of whole tiles
        // started together do; those shapes keep whole tiles.  It also loses when the reduction is short: 1024 x 2048 x 2048
        // (32 tiles, 14 chunks per pair) 130 as whole tiles with the last round split -> 113; taken from 32 chunks per pair.
        // g_stream_k (test hook): 1 = always, -1 = never.
        // With no more tiles than pairs the kernel still pays (one round, split along K when at most half the pairs have a
        // tile): its epilogue stores straight from registers -- 1536^3 113 -> 130, 2048^3 196 -> 208 TFLOP/s against one
        // tile per pair launch.
        const long long total_chunks = static_cast<long long>(T) * nch;
        const bool streamk = P > 0 && g_stream_k >= 0 && total_chunks >= 2 &&
                             (g_stream_k == 1 || (2 * T <= P && total_chunks >= 32LL * P));
        if (P > 0)
        {
            PersistPlan plan;
            plan.tiles_m = tiles_m, plan.tiles_n = tiles_n;
            plan.num_kb   = num_kb;
            plan.chunk_kb = chunk_kb;
            plan.full_units = T, plan.split_tiles = 0, plan.kb_mid = 0, plan.partial = nullptr, plan.tickets = nullptr;
            plan.counters = nullptr;
            plan.streamk = 0, plan.chunks_per_tile = nch, plan.max_parts = 2;
            const int R = T % P;
            if (streamk)
            {
                const int pairs_used = total_chunks < P ? static_cast<int>(total_chunks) : P;
                const long long per  = total_chunks / pairs_used;  // chunks of the shortest range (>= 1)
                if ((per + 1) / nch + 2 > kMaxSkUnits)
                {
                    set_last_error("gemm: stream-K range of %lld chunks over tiles of %d does not fit the unit list", per + 1, nch);
                    return kInvalidArgument;
                }
                plan.streamk   = 1;
                plan.max_parts = static_cast<int>((nch + per - 1) / per) + 1;
                if ((rc = tail_split_scratch(static_cast<size_t>(T) * plan.max_parts * 2 * kBM * BN, static_cast<size_t>(T) * 2)))
                    return rc;
                plan.partial = g_part, plan.tickets = g_tickets;
                P = pairs_used;
            }
            else if (g_persist_pairs >= 0 && (rc = unit_counters(&plan.counters)))  // (negative test-hook value: fixed assignment)
                return rc;
            if (!streamk && R > 0 && 2 * R <= P && plan.num_kb >= 4 * plan.chunk_kb)
            {
                plan.split_tiles = R;
                plan.full_units  = T - R;
                plan.kb_mid      = ((plan.num_kb / 2 + plan.chunk_kb - 1) / plan.chunk_kb) * plan.chunk_kb;
                if ((rc = tail_split_scratch(static_cast<size_t>(R) * 4 * kBM * BN, static_cast<size_t>(R) * 2)))
                    return rc;
                plan.partial = g_part, plan.tickets = g_tickets;
            }
            const int units = streamk ? P : plan.full_units + 2 * plan.split_tiles;
            cudaLaunchConfig_t cfg;
            std::memset(&cfg, 0, sizeof(cfg));
            cfg.gridDim          = dim3(static_cast<unsigned>(2 * (units < P ? units : P)), 1, 1);
            cfg.blockDim         = dim3(kThreads, 1, 1);
            cfg.dynamicSmemBytes = kPSmem;
            cfg.stream           = stream;
            cudaLaunchAttribute attr[1];
            attr[0].id               = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = 2;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = 1;
            cfg.attrs                = attr;
            cfg.numAttrs             = 1;
            GemmParams q   = p;
            q.kb_per_split = plan.num_kb;
            cudaError_t e  = cudaLaunchKernelEx(&cfg, gemm_tc2_persistent_kernel, tm, q, a_mn, b_mn, plan);
            ++g_launch_count;
            if (e != cudaSuccess)
            {
                set_last_error("gemm_tc2_persistent_kernel launch failed: %s", cudaGetErrorString(e));
                return kCudaError;
            }
            return kOk;
        }
    }
    int slabs = (terms == 1 && p.K >= 8 * kBK) ? 2 : 1;
    if (g_slabs == 1 || g_slabs == 2)
        slabs = terms == 1 ? g_slabs : 1;
    const int stages = Cfg::stages(terms) / slabs;
    const int smem   = Cfg::smem_bytes(terms);
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    dev &= 63;
    if (!attr_set[dev])
    {
        const int mx = Cfg::smem_bytes(1) > Cfg::smem_bytes(3) ? Cfg::smem_bytes(1) : Cfg::smem_bytes(3);
        cudaError_t e = cudaFuncSetAttribute(gemm_tc2_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, mx);
        if (e != cudaSuccess)
        {
            set_last_error("cudaFuncSetAttribute(pair kernel, smem=%d) failed: %s", mx, cudaGetErrorString(e));
            return kCudaError;
        }
        attr_set[dev] = true;
    }
    GemmParams q   = p;
    const int num_kb = (p.K + kBK * slabs - 1) / (kBK * slabs);
    q.kb_per_split   = num_kb;
    int chunk_kb     = g_chunk_kb > 0 ? (g_chunk_kb + slabs - 1) / slabs : (terms == 3 ? 64 / kBK : num_kb);
    if (chunk_kb > num_kb)
        chunk_kb = num_kb;
    const int pairs = ((p.M + 2 * kBM - 1) / (2 * kBM)) * ((p.N + BN - 1) / BN);
    cudaLaunchConfig_t cfg;
    std::memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim          = dim3(2 * pairs, 1, 1);
    cfg.blockDim         = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream           = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id               = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs                = attr;
    cfg.numAttrs             = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc2_kernel<BN>, tm, q, a_mn, b_mn, terms, stages, chunk_kb, slabs);
    ++g_launch_count;
    if (e != cudaSuccess)
    {
        set_last_error("gemm_tc2_kernel launch failed: %s", cudaGetErrorString(e));
        return kCudaError;
    }
    return kOk;
}

}  // namespace odl
