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

// acc: this thread's row (m0 + 32q + lane) x WARP_COLS columns starting at tile column cw.  stg: this warp's slab.
// BN is the tile width (the NCHW path is compiled for BN <= 128 only, see the launcher).
template <int BN, int WARP_COLS>
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
                    *reinterpret_cast<float4 *>(&stg[lane * kStgLd + 4 * i]) = v;
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
                    float4 v4     = *reinterpret_cast<const float4 *>(&stg[row * kStgLd + 4 * cg]);
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

}  // namespace odl
