// Inline-PTX wrappers for the sm_100a features the GEMM kernels use: mbarrier, TMA tiled loads,
// tcgen05 (TMEM allocation, MMA issue, commit, TMEM loads) and the fences between the async and
// generic proxies.  Every wait in this file is bounded: a wait that does not complete within
// ODL_WAIT_NS nanoseconds returns false so the caller can raise an error code and leave cleanly.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace odl
{
namespace ptx
{

#ifndef ODL_WAIT_NS
#define ODL_WAIT_NS 2000000000ull  // 2 s: far above any legitimate wait inside one CTA
#endif

__device__ __forceinline__ uint32_t smem_u32(const void *p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t globaltimer_ns()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ bool elect_one()
{
    uint32_t pred = 0;
    asm volatile(
        "{\n\t"
        ".reg .pred P;\n\t"
        "elect.sync _|P, 0xffffffff;\n\t"
        "selp.b32 %0, 1, 0, P;\n\t"
        "}\n"
        : "=r"(pred));
    return pred != 0;
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_mbar_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred P;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, P;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// try_wait with an explicit suspend-time hint: the thread may sleep in hardware until the phase completes or the hint
// (nanoseconds) runs out, instead of returning after the short default limit.  For waits of warps that share an SM
// with instruction-bound work, where a polling loop would take the issue slots that work needs.
__device__ __forceinline__ bool mbar_try_wait_hint(uint64_t *bar, uint32_t parity, uint32_t hint_ns)
{
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred P;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2, %3;\n\t"
        "selp.b32 %0, 1, 0, P;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(hint_ns)
        : "memory");
    return ok != 0;
}

// Bounded wait for long waits on a busy SM: suspends in hardware (20 us per try) and sleeps between tries.
__device__ __forceinline__ bool mbar_wait_quiet(uint64_t *bar, uint32_t parity, volatile int *abort_flag)
{
    if (mbar_try_wait(bar, parity))
        return true;
    const uint64_t t0 = globaltimer_ns();
    while (true)
    {
        if (mbar_try_wait_hint(bar, parity, 20000u))
            return true;
        __nanosleep(64);
        if (abort_flag && *abort_flag)
            return false;
        if (globaltimer_ns() - t0 > ODL_WAIT_NS)
        {
            if (abort_flag)
                *abort_flag = 1;
            return false;
        }
    }
}

// Bounded wait.  `abort_flag` (shared memory, may be null) lets one role's time-out release the others.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag)
{
    if (mbar_try_wait(bar, parity))
        return true;
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins    = 0;
    while (true)
    {
        if (mbar_try_wait(bar, parity))
            return true;
        if ((++spins & 0xff) == 0)
        {
            if (abort_flag && *abort_flag)
                return false;
            if (globaltimer_ns() - t0 > ODL_WAIT_NS)
            {
                if (abort_flag)
                    *abort_flag = 1;
                return false;
            }
        }
    }
}

// The same bounded wait with acquire semantics at CLUSTER scope: for a barrier whose arrival publishes data that the
// other CTA of the pair wrote into this CTA's shared memory (st.shared::cluster before a release.cluster arrive).
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t *bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred P;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 P, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, P;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

__device__ __forceinline__ bool mbar_wait_cluster(uint64_t *bar, uint32_t parity, volatile int *abort_flag)
{
    if (mbar_try_wait_cluster(bar, parity))
        return true;
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins    = 0;
    while (true)
    {
        if (mbar_try_wait_cluster(bar, parity))
            return true;
        if ((++spins & 0xff) == 0)
        {
            if (abort_flag && *abort_flag)
                return false;
            if (globaltimer_ns() - t0 > ODL_WAIT_NS)
            {
                if (abort_flag)
                    *abort_flag = 1;
                return false;
            }
        }
    }
}

// ---------------------------------------------------------------- proxies / fences
__device__ __forceinline__ void fence_proxy_async_smem()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_before_sync()
{
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after_sync()
{
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---------------------------------------------------------------- TMA (tiled loads, no multicast)
__device__ __forceinline__ void prefetch_tmap(const void *tmap)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}

// 2-D tile load global -> this CTA's shared memory, completion counted in bytes on `bar`.
// c0 is the innermost (contiguous) coordinate: c0 * 4 bytes must be a multiple of 16.
__device__ __forceinline__ void tma_load_2d(void *smem_dst, const void *tmap, uint64_t *bar, int32_t c0, int32_t c1)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        :
        : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}

// 3-D tile load (used for MN-major operands: {32 mn, k, mn / 32} moves several 32 x 32 boxes with one instruction).
__device__ __forceinline__ void tma_load_3d(void *smem_dst, const void *tmap, uint64_t *bar, int32_t c0, int32_t c1, int32_t c2)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        :
        : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

// ---------------------------------------------------------------- TMEM allocation (one warp, .sync.aligned)
__device__ __forceinline__ void tmem_alloc(uint32_t *smem_result, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
                 "r"(ncols)
                 : "memory");
}

__device__ __forceinline__ void tmem_relinquish()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// ---------------------------------------------------------------- tcgen05.mma (kind::tf32, A and B from shared memory)
// D[tmem] (+)= A[smem desc] * B[smem desc]; `accumulate` == 0 overwrites D.
__device__ __forceinline__ void mma_tf32_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                            uint32_t accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        :
        : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Make `bar` complete once every tcgen05.mma issued so far by this thread has finished.
__device__ __forceinline__ void mma_commit(uint64_t *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// ---------------------------------------------------------------- TMEM -> registers
// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp receives lane (base_lane + t), columns c..c+31.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_ld_wait()
{
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---------------------------------------------------------------- descriptors
// Shared-memory matrix descriptor, Blackwell version field = 1.
//   bits [0,14)  start address >> 4        bits [16,30) leading byte offset >> 4
//   bits [32,46) stride byte offset >> 4   bits [46,48) version (1)
//   bits [61,64) layout: 2 = SWIZZLE_128B (16-byte chunks; K-major operands),
//                        1 = SWIZZLE_128B with 32-byte chunks (the only layout MN-major 32-bit operands may use)
constexpr uint32_t kLayoutSw128      = 2;
constexpr uint32_t kLayoutSw64       = 4;  // 64-byte swizzle (16-byte chunks), K-major rows of 16 fp32
constexpr uint32_t kLayoutSw128Base32 = 1;
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                                   uint32_t layout)
{
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3fff);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fff) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fff) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(layout & 7) << 61;
    return d;
}

// Instruction descriptor for kind::tf32 with fp32 accumulation.
//   [4,6) D format (1 = f32)  [7,10) A format (2 = tf32)  [10,13) B format (2 = tf32)
//   bit 15 A is MN-major   bit 16 B is MN-major   [17,23) N >> 3   [24,29) M >> 4
__host__ __device__ constexpr uint32_t make_idesc_tf32(int m, int n, bool a_mn_major, bool b_mn_major)
{
    return (1u << 4) | (2u << 7) | (2u << 10) | ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16) |
           (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// ---------------------------------------------------------------- CTA pairs (cluster of 2, tcgen05 cta_group::2)
__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

// Address of the same shared-memory location in CTA `rank` of the cluster (shared::cluster window).
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}

__device__ __forceinline__ uint32_t ld_shared_cluster_u32(uint32_t cluster_addr)
{
    uint32_t v;
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(cluster_addr) : "memory");
    return v;
}

__device__ __forceinline__ void st_shared_cluster_u32(uint32_t cluster_addr, uint32_t v)
{
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}

__device__ __forceinline__ void st_shared_cluster_f32(uint32_t cluster_addr, float v)
{
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(cluster_addr), "f"(v) : "memory");
}

__device__ __forceinline__ void cluster_sync()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Arrive on a barrier that may live in the other CTA of the pair (shared::cluster address).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// The same arrive without release semantics: it does not wait for the thread's earlier global stores to be performed (a
// release at cluster scope does, which costs an epilogue warp a round trip to L2 behind every tile it has just written).
// For signals that publish no memory: "this TMEM buffer has been read" (ordered by tcgen05.wait::ld and the tcgen05
// fences), "this mailbox slot has been read" -- `after` is a value the arrive must follow (the word just read from the
// slot): the move makes the arrive wait for the load that produced it.
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t cluster_addr, uint32_t after = 0)
{
    asm volatile(
        "{\n\t"
        ".reg .b32 t;\n\t"
        "mov.b32 t, %1;\n\t"
        "mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];\n\t"
        "}" ::"r"(cluster_addr),
        "r"(after)
        : "memory");
}

__device__ __forceinline__ void tmem_alloc_pair(uint32_t *smem_result, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
                 "r"(ncols)
                 : "memory");
}

__device__ __forceinline__ void tmem_relinquish_pair()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// Tile load into THIS CTA's shared memory whose byte count is reported to a barrier of either CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(void *smem_dst, const void *tmap, uint32_t bar_cluster_addr, int32_t c0,
                                                 int32_t c1)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], "
        "[%2];"
        :
        : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
        : "memory");
}

__device__ __forceinline__ void tma_load_3d_pair(void *smem_dst, const void *tmap, uint32_t bar_cluster_addr, int32_t c0,
                                                 int32_t c1, int32_t c2)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], "
        "[%2];"
        :
        : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar_cluster_addr), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

// One MMA over both CTAs of the pair (M = 256: rows 0..127 accumulate in the leader's TMEM, 128..255 in its peer's;
// each CTA supplies its 128 rows of A and its half of B's rows from the same shared-memory offsets).
__device__ __forceinline__ void mma_tf32_ss_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                 uint32_t accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        :
        : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Completion of every pair-MMA issued so far -> one arrival on a barrier of either CTA (shared::cluster address).
__device__ __forceinline__ void mma_commit_pair(uint32_t bar_cluster_addr)
{
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr)
                 : "memory");
}

// The same, signalling the barrier at this shared-memory offset in BOTH CTAs of the pair with one instruction (the
// commit form with a CTA mask; it signals barriers only and moves no data).  One commit instead of two per stage
// release matters: every commit costs the tensor pipe on the order of a hundred idle cycles.
__device__ __forceinline__ void mma_commit_pair_both(uint64_t *bar)
{
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                     smem_u32(bar)),
                 "h"(mask)
                 : "memory");
}

}  // namespace ptx
}  // namespace odl
