// Operand preparation pass for the TF32 GEMMs (HBM-bound, one read of the source):
//   v = src[r,c]                                  (optionally v = aux[r,c] > 0 ? v : 0  -- ReLU backward mask)
//   dst_big[r,c]   = v                            (optional: a 16-byte-aligned, padded copy for the tiled loads)
//   dst_small[r,c] = tf32(v - trunc_tf32(v))      (optional: low part of the 3xTF32 split)
//   colsum[c]     += sum_r v                      (optional: bias gradient; per-slab partial sums are combined in a
//                                                  fixed order by the last block of a column group, so the result
//                                                  does not depend on block scheduling: same bits every run)
// Rows are walked by warps, columns by lanes in 128-bit groups, so every global access is a coalesced float4
// whenever pointer and pitch allow it; ragged edges and unaligned pitches fall back to scalar accesses.
#include <cuda_runtime.h>

#include "gemm_tc.cuh"
#include "host_util.h"
#include "internal.h"

namespace odl
{

namespace
{

constexpr int kSplitWarps = 8;
constexpr int kSplitRows  = 64;  // rows per block (256 for tall matrices: fewer slabs for the column sums' last step)

struct SplitParams
{
    const float *src;
    const float *aux;
    float *dst_big;
    float *dst_small;
    float *colsum;
    float *partial;    // [gridDim.y][gridDim.x * 128] per-slab column sums (only with colsum)
    unsigned *done;    // [gridDim.x] slabs finished per column group; left at zero by the launch
    int64_t ld_src, ld_aux, ld_dst;
    int rows, cols;
    int rows_per_block;
};

__global__ void __launch_bounds__(kSplitWarps * 32) split_kernel(const SplitParams p)
{
    __shared__ float red[kSplitWarps][32 * 4 + 4];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int c    = (blockIdx.x * 32 + lane) * 4;
    const int r0   = blockIdx.y * p.rows_per_block;
    const int r1   = min(r0 + p.rows_per_block, p.rows);

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
        const int64_t pitch = static_cast<int64_t>(gridDim.x) * 128;
        if (warp == 0)
        {
            float4 s4;
            float *sp = &s4.x;
#pragma unroll
            for (int j = 0; j < 4; ++j)
            {
                float s = 0.f;
#pragma unroll
                for (int w = 0; w < kSplitWarps; ++w)
                    s += red[w][lane * 4 + j];
                sp[j] = s;
            }
            *reinterpret_cast<float4 *>(p.partial + blockIdx.y * pitch + blockIdx.x * 128 + lane * 4) = s4;
            __threadfence();
        }
        // the last block of this column group to finish adds up all slabs, always in slab order
        __shared__ bool last;
        __syncthreads();
        if (threadIdx.x == 0)
        {
            __threadfence();
            last = atomicAdd(p.done + blockIdx.x, 1u) == gridDim.y - 1;
        }
        __syncthreads();
        if (!last)
            return;
        __threadfence();
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
        for (int y = warp; y < static_cast<int>(gridDim.y); y += kSplitWarps)
        {
            const float4 t = __ldcg(reinterpret_cast<const float4 *>(p.partial + y * pitch + blockIdx.x * 128 + lane * 4));
            acc.x += t.x, acc.y += t.y, acc.z += t.z, acc.w += t.w;
        }
        red[warp][lane * 4 + 0] = acc.x, red[warp][lane * 4 + 1] = acc.y;
        red[warp][lane * 4 + 2] = acc.z, red[warp][lane * 4 + 3] = acc.w;
        __syncthreads();
        if (warp == 0)
        {
#pragma unroll
            for (int j = 0; j < 4; ++j)
            {
                float s = 0.f;
#pragma unroll
                for (int w = 0; w < kSplitWarps; ++w)
                    s += red[w][lane * 4 + j];
                if (c + j < p.cols)
                    p.colsum[c + j] += s;
            }
        }
        if (threadIdx.x == 0)
            p.done[blockIdx.x] = 0;
    }
}

}  // namespace

namespace
{
// Scratch of the column sums: grown on demand (the device is drained first, like the scratch arena), never shrunk.
float *g_partial        = nullptr;
size_t g_partial_floats = 0;
unsigned *g_done        = nullptr;
size_t g_done_count     = 0;

int colsum_scratch(size_t floats, size_t groups)
{
    if (floats > g_partial_floats || groups > g_done_count)
    {
        if (cudaDeviceSynchronize() != cudaSuccess)
            return kCudaError;
        cudaFree(g_partial);
        cudaFree(g_done);
        g_partial = nullptr, g_done = nullptr, g_partial_floats = 0, g_done_count = 0;
        floats = floats + (floats >> 2);
        groups = groups < 1024 ? 1024 : 2 * groups;
        if (cudaMalloc(&g_partial, floats * 4) != cudaSuccess || cudaMalloc(&g_done, groups * 4) != cudaSuccess ||
            cudaMemset(g_done, 0, groups * 4) != cudaSuccess)
        {
            set_last_error("split: cannot allocate %zu bytes of column-sum scratch", floats * 4 + groups * 4);
            return kCudaError;
        }
        g_partial_floats = floats, g_done_count = groups;
        bump_scratch_generation();
    }
    return kOk;
}
}  // namespace

// Second half of the GEMM epilogue's column sums: colsum[n] += sum over slabs of partial[slab][n], slabs taken in a
// fixed order (8 interleaved chains, then the chains in order).
namespace
{
__global__ void __launch_bounds__(256) colsum_finish_kernel(const float *__restrict__ partial, int slabs, int64_t pitch,
                                                            int n_cols, float *__restrict__ colsum)
{
    __shared__ float red[8][33];
    const int lane = threadIdx.x & 31, chain = threadIdx.x >> 5;
    const int n = blockIdx.x * 32 + lane;
    float s     = 0.f;
    if (n < n_cols)
#pragma unroll 8
        for (int y = chain; y < slabs; y += 8)
            s += __ldcg(partial + y * pitch + n);
    red[chain][lane] = s;
    __syncthreads();
    if (chain == 0 && n < n_cols)
    {
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w)
            t += red[w][lane];
        colsum[n] += t;
    }
}
// The same sum for a slice buffer that holds two results side by side (columns [0, n_a) go to out_a, the next n_b to
// out_b); the results are assigned, not added: one launch, no zeroing of the outputs beforehand.
__global__ void __launch_bounds__(256) colsum_finish2_kernel(const float *__restrict__ partial, int slabs, int64_t pitch, int n_a,
                                                             float *__restrict__ out_a, int n_b, float *__restrict__ out_b)
{
    __shared__ float red[8][33];
    const int lane = threadIdx.x & 31, chain = threadIdx.x >> 5;
    const int n = blockIdx.x * 32 + lane;
    float s     = 0.f;
    if (n < n_a + n_b)
#pragma unroll 8
        for (int y = chain; y < slabs; y += 8)
            s += __ldcg(partial + y * pitch + n);
    red[chain][lane] = s;
    __syncthreads();
    if (chain == 0 && n < n_a + n_b)
    {
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w)
            t += red[w][lane];
        if (n < n_a)
            out_a[n] = t;
        else
            out_b[n - n_a] = t;
    }
}
}  // namespace

int colsum_finish2_launch(const float *partial, int slabs, int64_t pitch, int n_a, float *out_a, int n_b, float *out_b,
                          cudaStream_t stream)
{
    if (!out_b)
        n_b = 0;
    colsum_finish2_kernel<<<(n_a + n_b + 31) / 32, 256, 0, stream>>>(partial, slabs, pitch, n_a, out_a, n_b, out_b);
    ++g_launch_count;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
    {
        set_last_error("colsum_finish2_kernel launch failed: %s", cudaGetErrorString(e));
        return kCudaError;
    }
    return kOk;
}

float *colsum_partial_scratch(int slabs, int64_t pitch)
{
    return colsum_scratch(static_cast<size_t>(slabs) * pitch, 1) == kOk ? g_partial : nullptr;
}

int colsum_finish_launch(const float *partial, int slabs, int64_t pitch, int n_cols, float *colsum, cudaStream_t stream)
{
    colsum_finish_kernel<<<(n_cols + 31) / 32, 256, 0, stream>>>(partial, slabs, pitch, n_cols, colsum);
    ++g_launch_count;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
    {
        set_last_error("colsum_finish_kernel launch failed: %s", cudaGetErrorString(e));
        return kCudaError;
    }
    return kOk;
}

// colsum (if given) must be initialised by the caller (zeros for a plain sum); this pass adds to it.
int split_launch(const float *src, int64_t ld_src, int rows, int cols, const float *aux, int64_t ld_aux, float *dst_big,
                 float *dst_small, int64_t ld_dst, float *colsum, cudaStream_t stream)
{
    if (!src || rows <= 0 || cols <= 0)
    {
        set_last_error("split: invalid argument (rows=%d cols=%d)", rows, cols);
        return kInvalidArgument;
    }
    const int gx  = (cols + 127) / 128;
    const int rpb = (colsum && rows >= 32768 && static_cast<int64_t>(gx) * (rows / (4 * kSplitRows)) >= 148 * 8) ? 4 * kSplitRows : kSplitRows;
    dim3 grid(gx, (rows + rpb - 1) / rpb);
    if (colsum)
    {
        const int rc = colsum_scratch(static_cast<size_t>(grid.x) * 128 * grid.y, grid.x);
        if (rc)
            return rc;
    }
    SplitParams p{src, aux, dst_big, dst_small, colsum, g_partial, g_done, ld_src, ld_aux, ld_dst, rows, cols, rpb};
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
