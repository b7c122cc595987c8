// Operand preparation pass for the TF32 GEMMs (HBM-bound, one read of the source):
//   v = src[r,c]                                  (optionally v = aux[r,c] > 0 ? v : 0  -- ReLU backward mask)
//   dst_big[r,c]   = v                            (optional: a 16-byte-aligned, padded copy for the tiled loads)
//   dst_small[r,c] = tf32(v - trunc_tf32(v))      (optional: low part of the 3xTF32 split)
//   colsum[c]     += sum_r v                      (optional: bias gradient, fp32 atomics per 64-row slab)
// Rows are walked by warps, columns by lanes in 128-bit groups, so every global access is a coalesced float4
// whenever pointer and pitch allow it; ragged edges and unaligned pitches fall back to scalar accesses.
#include <cuda_runtime.h>

#include "gemm_tc.cuh"
#include "host_util.h"

namespace odl
{

namespace
{

constexpr int kSplitWarps = 8;
constexpr int kSplitRows  = 64;  // rows per block

struct SplitParams
{
    const float *src;
    const float *aux;
    float *dst_big;
    float *dst_small;
    float *colsum;
    int64_t ld_src, ld_aux, ld_dst;
    int rows, cols;
};

__global__ void __launch_bounds__(kSplitWarps * 32) split_kernel(const SplitParams p)
{
    __shared__ float red[kSplitWarps][32 * 4 + 4];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int c    = (blockIdx.x * 32 + lane) * 4;
    const int r0   = blockIdx.y * kSplitRows;
    const int r1   = min(r0 + kSplitRows, p.rows);

    const bool vec_src = ((p.ld_src & 3) == 0) && ((reinterpret_cast<uintptr_t>(p.src) & 15) == 0);
    const bool vec_aux = p.aux && ((p.ld_aux & 3) == 0) && ((reinterpret_cast<uintptr_t>(p.aux) & 15) == 0);
    const bool vec_dst = ((p.ld_dst & 3) == 0) && (!p.dst_big || (reinterpret_cast<uintptr_t>(p.dst_big) & 15) == 0) &&
                         (!p.dst_small || (reinterpret_cast<uintptr_t>(p.dst_small) & 15) == 0);
    const bool full4 = c + 3 < p.cols;

    float cs[4] = {0.f, 0.f, 0.f, 0.f};
    if (c < p.cols)
    {
        for (int r = r0 + warp; r < r1; r += kSplitWarps)
        {
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            const float *sp = p.src + static_cast<int64_t>(r) * p.ld_src + c;
            if (vec_src && full4)
            {
                const float4 t = __ldg(reinterpret_cast<const float4 *>(sp));
                v[0] = t.x, v[1] = t.y, v[2] = t.z, v[3] = t.w;
            }
            else
            {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (c + j < p.cols)
                        v[j] = __ldg(sp + j);
            }
            if (p.aux)
            {
                float a[4] = {0.f, 0.f, 0.f, 0.f};
                const float *ap = p.aux + static_cast<int64_t>(r) * p.ld_aux + c;
                if (vec_aux && full4)
                {
                    const float4 t = __ldg(reinterpret_cast<const float4 *>(ap));
                    a[0] = t.x, a[1] = t.y, a[2] = t.z, a[3] = t.w;
                }
                else
                {
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        if (c + j < p.cols)
                            a[j] = __ldg(ap + j);
                }
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    v[j] = a[j] > 0.f ? v[j] : 0.f;
            }
#pragma unroll
            for (int j = 0; j < 4; ++j)
                cs[j] += v[j];
            const int64_t o = static_cast<int64_t>(r) * p.ld_dst + c;
            if (vec_dst && full4)
            {
                if (p.dst_big)
                    *reinterpret_cast<float4 *>(p.dst_big + o) = make_float4(v[0], v[1], v[2], v[3]);
                if (p.dst_small)
                    *reinterpret_cast<float4 *>(p.dst_small + o) =
                        make_float4(tf32_small(v[0]), tf32_small(v[1]), tf32_small(v[2]), tf32_small(v[3]));
            }
            else
            {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (c + j < p.cols)
                    {
                        if (p.dst_big)
                            p.dst_big[o + j] = v[j];
                        if (p.dst_small)
                            p.dst_small[o + j] = tf32_small(v[j]);
                    }
            }
        }
    }
    if (p.colsum)
    {
#pragma unroll
        for (int j = 0; j < 4; ++j)
            red[warp][lane * 4 + j] = cs[j];
        __syncthreads();
        if (warp == 0 && c < p.cols)
        {
#pragma unroll
            for (int j = 0; j < 4; ++j)
            {
                float s = 0.f;
#pragma unroll
                for (int w = 0; w < kSplitWarps; ++w)
                    s += red[w][lane * 4 + j];
                if (c + j < p.cols)
                    atomicAdd(p.colsum + c + j, s);
            }
        }
    }
}

}  // namespace

// colsum (if given) must be zeroed by the caller; this pass only adds to it.
int split_launch(const float *src, int64_t ld_src, int rows, int cols, const float *aux, int64_t ld_aux, float *dst_big,
                 float *dst_small, int64_t ld_dst, float *colsum, cudaStream_t stream)
{
    if (!src || rows <= 0 || cols <= 0)
    {
        set_last_error("split: invalid argument (rows=%d cols=%d)", rows, cols);
        return kInvalidArgument;
    }
    SplitParams p{src, aux, dst_big, dst_small, colsum, ld_src, ld_aux, ld_dst, rows, cols};
    dim3 grid((cols + 127) / 128, (rows + kSplitRows - 1) / kSplitRows);
    split_kernel<<<grid, kSplitWarps * 32, 0, stream>>>(p);
    ++g_launch_count;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
    {
        set_last_error("split_kernel launch failed: %s", cudaGetErrorString(e));
        return kCudaError;
    }
    return kOk;
}

}  // namespace odl
