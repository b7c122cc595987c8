// Epilogue of the tcgen05 GEMM kernels, shared by the 1-CTA and the 2-CTA variants: takes one warp's accumulator
// slice out of registers (WARP_COLS columns of 32 rows), transposes it through a padded shared-memory slab and applies
//   + bias[n] -> ReLU -> ReLU-mask (aux > 0) -> per-slab column sums -> store D (+ low TF32 part), or the NCHW scatter store
// of conv outputs, or the store of a split-K partial tile into its slice, with coalesced 128-bit global accesses.
#pragma once
#include <cuda_runtime.h>

#include "gemm_tc.cuh"

namespace odl
{

constexpr int kStgLd = 36;  // padded row length (floats) of the per-warp 32 x 32 transpose slab

// Offset (floats) of the 16-byte chunk `chunk` (0..7) of row `row` inside a warp's transpose slab.  Two layouts, both free
// of bank conflicts for the quarter-warp phases of 128-bit accesses: rows padded to kStgLd floats (4608 B per slab), or,
// where shared memory is short (the persistent kernel keeps its slabs beside a live operand ring), unpadded 128-byte
// rows with the chunk index XOR-ed with the row (4096 B per slab).
template <bool SWZ>
__device__ __forceinline__ int slab_offset(int row, int chunk)
{
    return SWZ ? row * 32 + 4 * (chunk ^ (row & 7)) : row * kStgLd + 4 * chunk;
}

// acc: this thread's row (m0 + 32q + lane) x WARP_COLS columns starting at tile column cw.  stg: this warp's slab.
// BN is the tile width (the NCHW path is compiled for BN <= 128 only, see the launcher).
template <int BN, int WARP_COLS, bool SWZ = false>
__device__ __forceinline__ void gemm_epilogue_store(const GemmParams &p, float (&acc)[WARP_COLS], float *stg, int m0,
                                                    int n0, int cw, int q, int lane)
{
        // The last acc_full has fired, so every MMA has completed and every tile load was consumed: the operand
        // ring is dead and its first bytes now serve as per-warp transpose slabs (disjoint between warps).
            const int cg       = lane & 7;   // column group: columns 4cg..4cg+3 of the 32-column chunk
        const int rr       = lane >> 3;  // row offset 0..3
        const bool vec_d   = ((p.ldd & 3) == 0) && ((reinterpret_cast<uintptr_t>(p.D) & 15) == 0);
        const bool vec_s   = (p.flags & kEpiSmall) && ((reinterpret_cast<uintptr_t>(p.D_small) & 15) == 0);
        const bool vec_aux = (p.flags & kEpiMask) && ((p.ld_aux & 3) == 0) &&
                             ((reinterpret_cast<uintptr_t>(p.aux) & 15) == 0);
        if (BN <= 128 && (p.flags & kEpiNCHW))
        {
            // Conv output (the launcher never pairs this flag with the 256-wide tile): lanes hold consecutive rows m = consecutive pixels of one image, so for a fixed column
            // (output channel) a warp writes 32 consecutive floats of the NCHW tensor straight from registers.
            const int m = m0 + 32 * q + lane;
            if (m < p.M)
            {
                const int img = m / p.ohw;
                const int r   = m - img * p.ohw;
                float *dimg   = p.D + (static_cast<size_t>(img) * p.N) * p.ohw + r;
#pragma unroll
                for (int j = 0; j < (BN <= 128 ? WARP_COLS : 1); ++j)
                {
                    const int n = n0 + cw + j;
                    if (n < p.N)
                    {
                        float v = acc[j];
                        if (p.flags & kEpiScale)
                            v = __fmul_rn(v, __ldg(p.scale + n));
                        if (p.flags & kEpiBias)
                            v = __fadd_rn(v, __ldg(p.bias + n));
                        if (p.flags & kEpiRelu)
                            v = v > 0.f ? v : 0.f;
                        if (p.flags & kEpiSilu)
                            v = __fmul_rn(v, __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-v))));
                        dimg[static_cast<size_t>(n) * p.ohw] = v;
                    }
                }
            }
        }
        else
#pragma unroll
        for (int j = 0; j < WARP_COLS / 32; ++j)
        {
            const int c0 = cw + 32 * j;
            if (n0 + c0 < p.N)
            {
#pragma unroll
                for (int i = 0; i < 8; ++i)
                {
                    float4 v = make_float4(acc[32 * j + 4 * i], acc[32 * j + 4 * i + 1], acc[32 * j + 4 * i + 2],
                                           acc[32 * j + 4 * i + 3]);
                    *reinterpret_cast<float4 *>(&stg[slab_offset<SWZ>(lane, i)]) = v;
                }
                __syncwarp();

                const int n    = n0 + c0 + 4 * cg;
                float bias4[4] = {0.f, 0.f, 0.f, 0.f};
                if (p.flags & kEpiBias)
                {
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj)
                        if (n + jj < p.N)
                            bias4[jj] = __ldg(p.bias + n + jj);
                }
                float csum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int i = 0; i < 8; ++i)
                {
                    const int row = rr + 4 * i;
                    const int m   = m0 + 32 * q + row;
                    float4 v4     = *reinterpret_cast<const float4 *>(&stg[slab_offset<SWZ>(row, cg)]);
                    float v[4]    = {v4.x, v4.y, v4.z, v4.w};
                    if (m < p.M && n < p.N)
                    {
                        const bool full4 = (n + 3 < p.N);
                        if (p.flags & kEpiBias)
                        {
#pragma unroll
                            for (int jj = 0; jj < 4; ++jj)
                                v[jj] += bias4[jj];
                        }
                        if (p.flags & kEpiRelu)
                        {
#pragma unroll
                            for (int jj = 0; jj < 4; ++jj)
                                v[jj] = v[jj] > 0.f ? v[jj] : 0.f;
                        }
                        if (p.flags & kEpiMask)
                        {
                            const float *ap = p.aux + static_cast<size_t>(m) * p.ld_aux + n;
                            float a[4]      = {0.f, 0.f, 0.f, 0.f};
                            if (vec_aux && full4)
                            {
                                const float4 a4 = __ldg(reinterpret_cast<const float4 *>(ap));
                                a[0] = a4.x, a[1] = a4.y, a[2] = a4.z, a[3] = a4.w;
                            }
                            else
                            {
#pragma unroll
                                for (int jj = 0; jj < 4; ++jj)
                                    if (n + jj < p.N)
                                        a[jj] = __ldg(ap + jj);
                            }
#pragma unroll
                            for (int jj = 0; jj < 4; ++jj)
                                v[jj] = a[jj] > 0.f ? v[jj] : 0.f;
                        }
#pragma unroll
                        for (int jj = 0; jj < 4; ++jj)
                            if (n + jj < p.N)
                                csum[jj] += v[jj];
                        float *dp = p.D + static_cast<size_t>(m) * p.ldd + n;
                        if (p.flags & kEpiSplitK)
                            dp += static_cast<size_t>(blockIdx.y) * p.M * p.ldd;  // this split's slice of the scratch
                        if (vec_d && full4)
                        {
                            *reinterpret_cast<float4 *>(dp) = make_float4(v[0], v[1], v[2], v[3]);
                        }
                        else
                        {
#pragma unroll
                            for (int jj = 0; jj < 4; ++jj)
                                if (n + jj < p.N)
                                    dp[jj] = v[jj];
                        }
                        if (p.flags & kEpiSmall)
                        {
                            float *sp = p.D_small + static_cast<size_t>(m) * p.ldd + n;
                            if (vec_d && vec_s && full4)
                            {
                                *reinterpret_cast<float4 *>(sp) = make_float4(tf32_small(v[0]), tf32_small(v[1]),
                                                                              tf32_small(v[2]), tf32_small(v[3]));
                            }
                            else
                            {
#pragma unroll
                                for (int jj = 0; jj < 4; ++jj)
                                    if (n + jj < p.N)
                                        sp[jj] = tf32_small(v[jj]);
                            }
                        }
                    }
                }
                if (p.flags & kEpiColsum)
                {
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj)
                    {
                        csum[jj] += __shfl_xor_sync(0xffffffffu, csum[jj], 8);
                        csum[jj] += __shfl_xor_sync(0xffffffffu, csum[jj], 16);
                    }
                    if (rr == 0)
                    {
                        float *cp = p.colsum + static_cast<size_t>((m0 >> 5) + q) * p.ld_colsum + n;
#pragma unroll
                        for (int jj = 0; jj < 4; ++jj)
                            if (n + jj < p.N)
                                cp[jj] = csum[jj];
                    }
                }
                __syncwarp();
            }
        }
}

// ---- the same epilogue without the shared-memory round trip ------------------------------------------------------------
// For kernels whose epilogue runs while the tensor core is busy with the next tile: there the transpose slabs compete for
// shared-memory bandwidth with the operand ring (which already runs near the SM's limit), and the store phase takes
// longer than the MMA thread can run ahead.  Here every thread writes ITS row straight from registers with 256-bit
// stores: a warp instruction then covers 32 rows x 32 bytes = 32 full sectors, so L2 sees only whole sectors (four
// consecutive stores of a thread complete a 128-byte line) without any transposition.  Needs 32-byte aligned rows of D
// (ldd % 8 == 0); no column sums (they add over rows, i.e. across lanes -- the slab path keeps that case).
__device__ __forceinline__ void st_global_v8(float *ptr, const float (&v)[8])
{
    asm volatile("st.global.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(ptr), "f"(v[0]), "f"(v[1]), "f"(v[2]),
                 "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7])
                 : "memory");
}

__device__ __forceinline__ void ld_global_v8(const float *ptr, float (&v)[8])
{
    asm volatile("ld.global.v8.f32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7])
                 : "l"(ptr));
}

__host__ __device__ __forceinline__ bool epilogue_direct_ok(const GemmParams &p)
{
    if (p.flags & (kEpiNCHW | kEpiSplitK | kEpiScale | kEpiSilu))
        return false;
    if ((p.ldd & 7) || (reinterpret_cast<uintptr_t>(p.D) & 31))
        return false;
    if ((p.flags & kEpiSmall) && (reinterpret_cast<uintptr_t>(p.D_small) & 31))
        return false;
    if ((p.flags & kEpiMask) && ((p.ld_aux & 7) || (reinterpret_cast<uintptr_t>(p.aux) & 31)))
        return false;
    return true;
}

// Sum of v[c] over the 32 lanes of the warp for each of 32 columns c, delivered as: lane l returns the total of column l.
// A butterfly that halves every lane's set of columns per step (16 + 8 + 4 + 2 + 1 = 31 shuffles instead of 32 x 5): at
// the step with lane distance s, a lane keeps the half of its columns whose index bit s equals its own lane bit s, hands
// the other half to its partner and adds what the partner hands over.  The order of the additions is fixed.
__device__ __forceinline__ float warp_column_sums_32(float (&v)[32], int lane)
{
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1)
    {
        const bool upper = (lane & s) != 0;
#pragma unroll
        for (int i = 0; i < s; ++i)
        {
            const float lo = v[i], hi = v[i + s];
            const float recv = __shfl_xor_sync(0xffffffffu, upper ? lo : hi, s);
            v[i]             = (upper ? hi : lo) + recv;
        }
    }
    return v[0];
}

// acc: this thread's row (m0 + 32q + lane), WARP_COLS columns starting at tile column cw.  Every lane of the warp must
// call it (the column sums shuffle across all 32 lanes).
template <int WARP_COLS>
__device__ __forceinline__ void gemm_epilogue_direct(const GemmParams &p, float (&acc)[WARP_COLS], int m0, int n0, int cw,
                                                     int q, int lane)
{
    const int m        = m0 + 32 * q + lane;
    const bool row_ok  = m < p.M;
    float *drow        = p.D + static_cast<size_t>(m) * p.ldd;
    float *srow        = (p.flags & kEpiSmall) ? p.D_small + static_cast<size_t>(m) * p.ldd : nullptr;
    const float *arow  = (p.flags & kEpiMask) ? p.aux + static_cast<size_t>(m) * p.ld_aux : nullptr;
#pragma unroll
    for (int b = 0; b < WARP_COLS / 32; ++b)
    {
        const int nb = n0 + cw + 32 * b;
        if (nb >= p.N)
            break;  // uniform over the warp
        float(&blk)[32] = *reinterpret_cast<float(*)[32]>(&acc[32 * b]);  // finished in place: acc is dead afterwards
#pragma unroll
        for (int g = 0; g < 4; ++g)
        {
            const int n = nb + 8 * g;
            float(&v)[8] = *reinterpret_cast<float(*)[8]>(&acc[32 * b + 8 * g]);
            const bool full = n + 8 <= p.N;
            if (row_ok && n < p.N)
            {
                if (p.flags & kEpiBias)
                {
                    if (full)
                    {
                        const float4 b0 = __ldg(reinterpret_cast<const float4 *>(p.bias + n) + 0);
                        const float4 b1 = __ldg(reinterpret_cast<const float4 *>(p.bias + n) + 1);
                        v[0] += b0.x, v[1] += b0.y, v[2] += b0.z, v[3] += b0.w;
                        v[4] += b1.x, v[5] += b1.y, v[6] += b1.z, v[7] += b1.w;
                    }
                    else
                    {
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            if (n + j < p.N)
                                v[j] += __ldg(p.bias + n + j);
                    }
                }
                if (p.flags & kEpiRelu)
                {
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        v[j] = v[j] > 0.f ? v[j] : 0.f;
                }
                if (p.flags & kEpiMask)
                {
                    float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                    if (full)
                        ld_global_v8(arow + n, a);
                    else
                    {
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            if (n + j < p.N)
                                a[j] = __ldg(arow + n + j);
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        v[j] = a[j] > 0.f ? v[j] : 0.f;
                }
                if (full)
                {
                    st_global_v8(drow + n, v);
                    if (srow)
                    {
                        float sm[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            sm[j] = tf32_small(v[j]);
                        st_global_v8(srow + n, sm);
                    }
                }
                else
                {
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        if (n + j < p.N)
                        {
                            drow[n + j] = v[j];
                            if (srow)
                                srow[n + j] = tf32_small(v[j]);
                        }
                }
            }
            if (p.flags & kEpiColsum)
            {
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    v[j] = (row_ok && n + j < p.N) ? v[j] : 0.f;  // rows and columns outside the matrix add nothing
            }
        }
        if (p.flags & kEpiColsum)
        {
            // per-slab partial column sums (the launcher adds the slabs in order afterwards): lane l ends up with column l
            const float total = warp_column_sums_32(blk, lane);
            if (nb + lane < p.N)
                p.colsum[static_cast<size_t>((m0 >> 5) + q) * p.ld_colsum + nb + lane] = total;
        }
    }
}

}  // namespace odl
