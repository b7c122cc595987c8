// BatchNorm over x[N, C, HW] (HW = 1: the {N, C} form) with a fused ReLU / SiLU, forward and backward, and SiLU alone.
//
// Arithmetic follows the reference's CPU kernels (src/mat/origin/cpu/normalization/batch_norm.cpp:20-415,
// src/mat/origin/cpu/activation/silu.cpp:48-92): biased batch variance, x_norm = (x - mean) / sqrt(var + eps),
// y = gamma * x_norm + beta, every operation rounded to fp32 on its own (no fused multiply-add), so that with given
// statistics (evaluation mode) the forward is bit-identical.  The batch statistics themselves are reduced in double
// precision across blocks (the reference's single sequential fp32 accumulator has no parallel equivalent).
//
// What is NOT kept from the reference: the x_norm tensor it saves for backward (a full extra activation).  Backward
// recomputes x_norm and the pre-activation from x, the saved statistics, gamma and beta.
//
// All kernels are HBM-bound streaming passes: forward = 2 reads + 1 write of x, backward = 2 reads of (gy, x) + 1 write.
// Grids are (channel, slabs) with slabs chosen so that the grid is a few waves of the 148 SMs.
#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/odl_b200.h"
#include "gemm_tc.cuh"
#include "host_util.h"
#include "internal.h"

namespace odl
{
namespace
{
constexpr int kThreads = 256;

struct BnGeom
{
    int N, C, HW;
    int chunks;     // slabs per (n, c) plane (4-D form) or row slabs (2-D form)
    int chunk_len;  // elements of a plane per slab / rows per slab (a multiple of 4 in the 4-D form)
};

// Pre-activation -> activation and its derivative (act: 0 none, 1 relu, 2 silu), the reference's formulas.
__device__ __forceinline__ float act_forward(float z, int act)
{
    if (act == 1)
        return z > 0.f ? z : 0.f;
    if (act == 2)
    {
        const float s = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-z)));
        return __fmul_rn(z, s);
    }
    return z;
}
__device__ __forceinline__ float act_backward(float gy, float z, int act)
{
    if (act == 1)
        return z > 0.f ? gy : 0.f;
    if (act == 2)
    {
        const float s = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-z)));
        const float d = __fadd_rn(s, __fmul_rn(__fmul_rn(z, s), __fsub_rn(1.0f, s)));
        return __fmul_rn(gy, d);
    }
    return gy;
}

// Element range of one block: channel c = blockIdx.x; 4-D form: plane n = blockIdx.y / chunks, elements
// [i0, i1) of that plane; 2-D form (HW == 1): rows [i0, i1), element (n, c) at n * C + c.
struct Range
{
    const int64_t base;  // offset of element i = 0
    const int64_t step;  // distance between consecutive i
    const int i0, i1;
};
__device__ __forceinline__ Range block_range(const BnGeom &g)
{
    const int c = blockIdx.x;
    if (g.HW == 1)
    {
        const int r0 = blockIdx.y * g.chunk_len;
        const int r1 = min(g.N, r0 + g.chunk_len);
        return Range{static_cast<int64_t>(c), static_cast<int64_t>(g.C), r0, r1};
    }
    const int n  = blockIdx.y / g.chunks;
    const int k  = blockIdx.y - n * g.chunks;
    const int i0 = k * g.chunk_len;
    const int i1 = min(g.HW, i0 + g.chunk_len);
    return Range{(static_cast<int64_t>(n) * g.C + c) * g.HW, 1, i0, i1};
}

__device__ __forceinline__ void block_sum2(double &a, double &b)
{
    __shared__ double red[2][kThreads / 32];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
    {
        a += __shfl_xor_sync(0xffffffffu, a, o);
        b += __shfl_xor_sync(0xffffffffu, b, o);
    }
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    if (l == 0)
        red[0][w] = a, red[1][w] = b;
    __syncthreads();
    if (w == 0)
    {
        a = l < kThreads / 32 ? red[0][l] : 0.0;
        b = l < kThreads / 32 ? red[1][l] : 0.0;
#pragma unroll
        for (int o = 4; o > 0; o >>= 1)
        {
            a += __shfl_xor_sync(0xffffffffu, a, o);
            b += __shfl_xor_sync(0xffffffffu, b, o);
        }
    }
}

// One block's elements, V at a time (V = 4: float4 loads / stores; the launcher guarantees 16-byte alignment of every
// group then).  body(offset, lane values...) is written out per kernel below through these two helpers.
template <int V>
__device__ __forceinline__ void load_vec(const float *__restrict__ p, float (&v)[V])
{
    if (V == 4)
    {
        const float4 t = __ldg(reinterpret_cast<const float4 *>(p));
        v[0] = t.x, v[1] = t.y, v[2] = t.z, v[3] = t.w;
    }
    else
        v[0] = __ldg(p);
}
template <int V>
__device__ __forceinline__ void store_vec(float *__restrict__ p, const float (&v)[V])
{
    if (V == 4)
        *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
    else
        p[0] = v[0];
}

// Finishes a channel once its last block has stored its partial sums.  Called by every thread of the block with the
// block's sums in thread 0; returns true in exactly one thread of the grid per channel, with the totals in (s, q).
// No floating-point atomics: every block stores its pair into its own slot of acc[C][gridDim.y][2], and the block that
// arrives last adds the slots in a fixed order (thread t takes slots t, t + kThreads, ... ascending, then the fixed
// shuffle tree of block_sum2), so the statistics have the same bits on every run whatever order the blocks finish in.
__device__ __forceinline__ bool channel_done(double *acc, unsigned *done, int c, double &s, double &q)
{
    __shared__ int is_last;
    const int nb       = gridDim.y;
    double *slots      = acc + 2 * static_cast<int64_t>(c) * nb;
    if (threadIdx.x == 0)
    {
        slots[2 * blockIdx.y]     = s;
        slots[2 * blockIdx.y + 1] = q;
        __threadfence();
        is_last = atomicAdd(done + c, 1u) == static_cast<unsigned>(nb - 1) ? 1 : 0;
    }
    __syncthreads();
    if (!is_last)
        return false;
    __threadfence();
    double a = 0.0, b = 0.0;
    for (int i = threadIdx.x; i < nb; i += kThreads)
    {
        a += __ldcg(slots + 2 * i);
        b += __ldcg(slots + 2 * i + 1);
    }
    block_sum2(a, b);
    s = a, q = b;
    return threadIdx.x == 0;
}

// ---- forward, training: per-channel sum and sum of squares; the last block of a channel finishes the statistics
template <int V>
__global__ void __launch_bounds__(kThreads) bn_stats_kernel(const float *__restrict__ x, BnGeom g, double *__restrict__ acc,
                                                            unsigned *__restrict__ done, float *__restrict__ save_mean,
                                                            float *__restrict__ save_var, float *__restrict__ running_mean,
                                                            float *__restrict__ running_var, float momentum)
{
    const Range r = block_range(g);
    double s = 0.0, q = 0.0;
    for (int i = r.i0 + V * threadIdx.x; i < r.i1; i += V * kThreads)
    {
        float v[V];
        load_vec<V>(x + r.base + i * r.step, v);
#pragma unroll
        for (int j = 0; j < V; ++j)
        {
            const double d = static_cast<double>(v[j]);
            s += d;
            q += d * d;
        }
    }
    block_sum2(s, q);
    const int c = blockIdx.x;
    if (channel_done(acc, done, c, s, q))
    {
        const double count = static_cast<double>(g.N) * g.HW;
        const double mean  = s / count;
        double var         = q / count - mean * mean;
        var                = var > 0.0 ? var : 0.0;
        const float mf = static_cast<float>(mean), vf = static_cast<float>(var);
        save_mean[c] = mf;
        save_var[c]  = vf;
        if (running_mean)  // nn::BatchNorm2d: momentum weighs the OLD value (src/nn/layers/batch_norm2d.cpp:76-79)
        {
            const float keep = __fsub_rn(1.0f, momentum);
            running_mean[c]  = __fadd_rn(__fmul_rn(momentum, running_mean[c]), __fmul_rn(keep, mf));
            running_var[c]   = __fadd_rn(__fmul_rn(momentum, running_var[c]), __fmul_rn(keep, vf));
        }
    }
}

// ---- forward: y = act(gamma * (x - mean) / sqrt(var + eps) + beta), the reference's operation sequence
template <int V>
__global__ void __launch_bounds__(kThreads) bn_apply_kernel(const float *__restrict__ x, BnGeom g,
                                                            const float *__restrict__ gamma, const float *__restrict__ beta,
                                                            const float *__restrict__ mean, const float *__restrict__ var,
                                                            float eps, int act, float *__restrict__ y)
{
    const Range r = block_range(g);
    const int c   = blockIdx.x;
    const float m = mean[c], sd = __fsqrt_rn(__fadd_rn(var[c], eps)), ga = gamma[c], be = beta[c];
    for (int i = r.i0 + V * threadIdx.x; i < r.i1; i += V * kThreads)
    {
        const int64_t o = r.base + i * r.step;
        float v[V];
        load_vec<V>(x + o, v);
#pragma unroll
        for (int j = 0; j < V; ++j)
            v[j] = act_forward(__fadd_rn(__fmul_rn(ga, __fdiv_rn(__fsub_rn(v[j], m), sd)), be), act);
        store_vec<V>(y + o, v);
    }
}

// ---- backward: g = gy * act'(z); per-channel sum g and sum g * x_norm; the last block writes dgamma, dbeta and the
//      two means the second pass needs.  (x - mean) * (1 / std) here: no bit-level claim is made for gradients.
template <int V>
__global__ void __launch_bounds__(kThreads)
    bn_bwd_stats_kernel(const float *__restrict__ gy, const float *__restrict__ x, BnGeom g, const float *__restrict__ gamma,
                        const float *__restrict__ beta, const float *__restrict__ mean, const float *__restrict__ var,
                        float eps, int act, double *__restrict__ acc, unsigned *__restrict__ done,
                        float *__restrict__ dgamma, float *__restrict__ dbeta, float *__restrict__ means)
{
    const Range r = block_range(g);
    const int c   = blockIdx.x;
    const float m = mean[c], rsd = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var[c], eps))), ga = gamma[c], be = beta[c];
    double s = 0.0, q = 0.0;
    for (int i = r.i0 + V * threadIdx.x; i < r.i1; i += V * kThreads)
    {
        const int64_t o = r.base + i * r.step;
        float xv[V], gv[V];
        load_vec<V>(x + o, xv);
        load_vec<V>(gy + o, gv);
#pragma unroll
        for (int j = 0; j < V; ++j)
        {
            const float xn = __fmul_rn(__fsub_rn(xv[j], m), rsd);
            const float t  = act_backward(gv[j], __fadd_rn(__fmul_rn(ga, xn), be), act);
            s += static_cast<double>(t);
            q += static_cast<double>(__fmul_rn(t, xn));
        }
    }
    block_sum2(s, q);
    if (channel_done(acc, done, c, s, q))
    {
        const float sum_g = static_cast<float>(s), sum_q = static_cast<float>(q);
        const float count = static_cast<float>(static_cast<int64_t>(g.N) * g.HW);
        dbeta[c]          = sum_g;
        dgamma[c]         = sum_q;
        means[2 * c]      = __fdiv_rn(sum_g, count);
        means[2 * c + 1]  = __fdiv_rn(sum_q, count);
    }
}

// ---- backward: gx = (gamma / std) * (g - mean(g) - x_norm * mean(g * x_norm))
template <int V>
__global__ void __launch_bounds__(kThreads)
    bn_bwd_apply_kernel(const float *__restrict__ gy, const float *__restrict__ x, BnGeom g, const float *__restrict__ gamma,
                        const float *__restrict__ beta, const float *__restrict__ mean, const float *__restrict__ var,
                        float eps, int act, const float *__restrict__ means, float *__restrict__ gx)
{
    const Range r = block_range(g);
    const int c   = blockIdx.x;
    const float m = mean[c], sd = __fsqrt_rn(__fadd_rn(var[c], eps)), rsd = __fdiv_rn(1.0f, sd), ga = gamma[c], be = beta[c];
    const float k = __fdiv_rn(ga, sd), mg = means[2 * c], mq = means[2 * c + 1];
    for (int i = r.i0 + V * threadIdx.x; i < r.i1; i += V * kThreads)
    {
        const int64_t o = r.base + i * r.step;
        float xv[V], gv[V];
        load_vec<V>(x + o, xv);
        load_vec<V>(gy + o, gv);
#pragma unroll
        for (int j = 0; j < V; ++j)
        {
            const float xn = __fmul_rn(__fsub_rn(xv[j], m), rsd);
            const float t  = act_backward(gv[j], __fadd_rn(__fmul_rn(ga, xn), be), act);
            gv[j]          = __fmul_rn(k, __fsub_rn(__fsub_rn(t, mg), __fmul_rn(xn, mq)));
        }
        store_vec<V>(gx + o, gv);
    }
}

// ---- folding evaluation-mode BatchNorm into the epilogue of the GEMM that produces its input:
//      scale = gamma / sqrt(var + eps), shift = beta + scale * (bias - mean)
__global__ void bn_fold_kernel(const float *__restrict__ gamma, const float *__restrict__ beta,
                               const float *__restrict__ mean, const float *__restrict__ var,
                               const float *__restrict__ bias, float eps, int C, float *__restrict__ scale,
                               float *__restrict__ shift)
{
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C)
        return;
    const float s = __fdiv_rn(gamma[c], __fsqrt_rn(__fadd_rn(var[c], eps)));
    scale[c]      = s;
    shift[c]      = __fadd_rn(beta[c], __fmul_rn(s, __fsub_rn(bias ? bias[c] : 0.0f, mean[c])));
}

__global__ void silu_fwd_kernel(const float *__restrict__ x, float *__restrict__ y, int64_t n)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
        y[i] = act_forward(x[i], 2);
}
__global__ void silu_bwd_kernel(const float *__restrict__ gy, const float *__restrict__ x, float *__restrict__ gx, int64_t n)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
        gx[i] = act_backward(gy[i], x[i], 2);
}

int check_launch(const char *name)
{
    ++g_launch_count;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
    {
        set_last_error("%s launch failed: %s", name, cudaGetErrorString(e));
        return kCudaError;
    }
    return kOk;
}

// float4 access needs planes that start and end on 16-byte boundaries.
bool vec4_ok(const BnGeom &g, const void *a, const void *b)
{
    return g.HW > 1 && (g.HW & 3) == 0 && !(reinterpret_cast<uintptr_t>(a) & 15) && !(reinterpret_cast<uintptr_t>(b) & 15);
}

// Slabs: enough blocks for about four waves of 148 SMs, at least 1024 elements per block.
int make_geom(int64_t N, int64_t C, int64_t HW, BnGeom *g, dim3 *grid)
{
    if (N <= 0 || C <= 0 || HW <= 0 || N > 0x7fffffff || C > 0x7fffffff || HW > 0x7fffffff)
    {
        set_last_error("batch_norm: invalid shape (N=%lld C=%lld HW=%lld)", (long long)N, (long long)C, (long long)HW);
        return kInvalidArgument;
    }
    g->N = (int)N, g->C = (int)C, g->HW = (int)HW;
    const int64_t want = (4 * 148 + C - 1) / C;  // blocks per channel
    int64_t per_channel;
    if (HW == 1)
    {
        int64_t slabs = want < 1 ? 1 : want;
        int64_t len   = (N + slabs - 1) / slabs;
        if (len < 256)
            len = 256;
        g->chunk_len = (int)len;
        g->chunks    = (int)((N + len - 1) / len);
        per_channel  = g->chunks;
    }
    else
    {
        int64_t chunks = (want + N - 1) / N;
        if (chunks < 1)
            chunks = 1;
        int64_t len = (HW + chunks - 1) / chunks;
        if (len < 1024)
            len = 1024;
        len = (len + 3) & ~int64_t(3);
        g->chunk_len = (int)len;
        g->chunks    = (int)((HW + len - 1) / len);
        per_channel  = N * g->chunks;
    }
    if (per_channel > 65535)
    {
        // fewer, longer slabs: the y dimension of a grid holds 65535 blocks
        const int64_t shrink = (per_channel + 65534) / 65535;
        g->chunk_len *= (int)shrink;  // stays a multiple of 4
        g->chunks   = (int)(((HW == 1 ? N : HW) + g->chunk_len - 1) / g->chunk_len);
        per_channel = HW == 1 ? g->chunks : N * g->chunks;
        if (per_channel > 65535)
        {
            set_last_error("batch_norm: batch of %lld planes exceeds the grid", (long long)N);
            return kTooLarge;
        }
    }
    *grid = dim3((unsigned)C, (unsigned)per_channel);
    return kOk;
}
}  // namespace
}  // namespace odl

using namespace odl;
#define ST(x) static_cast<cudaStream_t>(x)

extern "C" {

int odl_batch_norm_forward(const float *x, const float *gamma, const float *beta, float *running_mean,
                           float *running_var, int training, float eps, float momentum, int64_t N, int64_t C, int64_t HW,
                           int act, float *y, float *save_mean, float *save_var, void *stream)
{
    if (!x || !gamma || !beta || !y || act < 0 || act > 2 || (!training && (!running_mean || !running_var)) ||
        (training && (!save_mean || !save_var)) || (!running_mean != !running_var))
    {
        set_last_error("batch_norm_forward: invalid argument (training=%d act=%d)", training, act);
        return kInvalidArgument;
    }
    BnGeom g;
    dim3 grid;
    int rc = make_geom(N, C, HW, &g, &grid);
    if (rc)
        return rc;
    cudaStream_t s    = ST(stream);
    const float *mean = running_mean, *var = running_var;
    if (training)
    {
        arena_reset();
        const size_t acc_bytes = sizeof(double) * 2 * C * grid.y, all = acc_bytes + sizeof(unsigned) * C;
        if ((rc = arena_reserve(all + 256)))
            return rc;
        double *acc    = static_cast<double *>(arena_alloc(acc_bytes));
        unsigned *done = static_cast<unsigned *>(arena_alloc(sizeof(unsigned) * C));
        ODL_CUDA_TRY(cudaMemsetAsync(done, 0, sizeof(unsigned) * C, s));
        if (vec4_ok(g, x, x))
            bn_stats_kernel<4><<<grid, kThreads, 0, s>>>(x, g, acc, done, save_mean, save_var, running_mean, running_var,
                                                         momentum);
        else
            bn_stats_kernel<1><<<grid, kThreads, 0, s>>>(x, g, acc, done, save_mean, save_var, running_mean, running_var,
                                                         momentum);
        if ((rc = check_launch("bn_stats_kernel")))
            return rc;
        mean = save_mean, var = save_var;
    }
    else if (save_mean && save_var)
    {
        ODL_CUDA_TRY(cudaMemcpyAsync(save_mean, running_mean, sizeof(float) * C, cudaMemcpyDeviceToDevice, s));
        ODL_CUDA_TRY(cudaMemcpyAsync(save_var, running_var, sizeof(float) * C, cudaMemcpyDeviceToDevice, s));
    }
    if (vec4_ok(g, x, y))
        bn_apply_kernel<4><<<grid, kThreads, 0, s>>>(x, g, gamma, beta, mean, var, eps, act, y);
    else
        bn_apply_kernel<1><<<grid, kThreads, 0, s>>>(x, g, gamma, beta, mean, var, eps, act, y);
    return check_launch("bn_apply_kernel");
}

int odl_batch_norm_backward(const float *gy, const float *x, const float *gamma, const float *beta, const float *save_mean,
                            const float *save_var, float eps, int64_t N, int64_t C, int64_t HW, int act, float *gx,
                            float *dgamma, float *dbeta, void *stream)
{
    if (!gy || !x || !gamma || !beta || !save_mean || !save_var || !gx || !dgamma || !dbeta || act < 0 || act > 2)
    {
        set_last_error("batch_norm_backward: invalid argument (act=%d)", act);
        return kInvalidArgument;
    }
    BnGeom g;
    dim3 grid;
    int rc = make_geom(N, C, HW, &g, &grid);
    if (rc)
        return rc;
    cudaStream_t s = ST(stream);
    arena_reset();
    const size_t acc_bytes = sizeof(double) * 2 * C * grid.y;
    if ((rc = arena_reserve(acc_bytes + sizeof(unsigned) * C + sizeof(float) * 2 * C + 512)))
        return rc;
    double *acc    = static_cast<double *>(arena_alloc(acc_bytes));
    unsigned *done = static_cast<unsigned *>(arena_alloc(sizeof(unsigned) * C));
    float *means   = static_cast<float *>(arena_alloc(sizeof(float) * 2 * C));
    ODL_CUDA_TRY(cudaMemsetAsync(done, 0, sizeof(unsigned) * C, s));
    const bool v4 = vec4_ok(g, x, gy) && vec4_ok(g, x, gx);
    if (v4)
        bn_bwd_stats_kernel<4><<<grid, kThreads, 0, s>>>(gy, x, g, gamma, beta, save_mean, save_var, eps, act, acc, done,
                                                         dgamma, dbeta, means);
    else
        bn_bwd_stats_kernel<1><<<grid, kThreads, 0, s>>>(gy, x, g, gamma, beta, save_mean, save_var, eps, act, acc, done,
                                                         dgamma, dbeta, means);
    if ((rc = check_launch("bn_bwd_stats_kernel")))
        return rc;
    if (v4)
        bn_bwd_apply_kernel<4><<<grid, kThreads, 0, s>>>(gy, x, g, gamma, beta, save_mean, save_var, eps, act, means, gx);
    else
        bn_bwd_apply_kernel<1><<<grid, kThreads, 0, s>>>(gy, x, g, gamma, beta, save_mean, save_var, eps, act, means, gx);
    return check_launch("bn_bwd_apply_kernel");
}

int odl_batch_norm_fold(const float *gamma, const float *beta, const float *mean, const float *var, const float *bias,
                        float eps, int64_t C, float *scale, float *shift, void *stream)
{
    if (!gamma || !beta || !mean || !var || !scale || !shift || C <= 0 || C > 0x7fffffff)
    {
        set_last_error("batch_norm_fold: invalid argument");
        return kInvalidArgument;
    }
    bn_fold_kernel<<<(unsigned)((C + 255) / 256), 256, 0, ST(stream)>>>(gamma, beta, mean, var, bias, eps, (int)C, scale,
                                                                        shift);
    return check_launch("bn_fold_kernel");
}

int odl_silu_forward(const float *x, float *y, int64_t n, void *stream)
{
    if (!x || !y || n <= 0)
    {
        set_last_error("silu_forward: invalid argument");
        return kInvalidArgument;
    }
    int64_t blocks = (n + 1023) / 1024;
    blocks         = blocks > 148 * 8 ? 148 * 8 : blocks;
    silu_fwd_kernel<<<(unsigned)blocks, 256, 0, ST(stream)>>>(x, y, n);
    return check_launch("silu_fwd_kernel");
}

int odl_silu_backward(const float *gy, const float *x, float *gx, int64_t n, void *stream)
{
    if (!gy || !x || !gx || n <= 0)
    {
        set_last_error("silu_backward: invalid argument");
        return kInvalidArgument;
    }
    int64_t blocks = (n + 1023) / 1024;
    blocks         = blocks > 148 * 8 ? 148 * 8 : blocks;
    silu_bwd_kernel<<<(unsigned)blocks, 256, 0, ST(stream)>>>(gy, x, gx, n);
    return check_launch("silu_bwd_kernel");
}

}  // extern "C"
