// HBM-bound kernels of the path: ReLU forward/backward, bias add, column sums, fused softmax-cross-entropy,
// fused Adam / SGD parameter updates, im2col / col2im and the NCHW <-> row-matrix permutations of Conv2d.
// All of them stream their operands once with 128-bit accesses where alignment allows and size their grids as a
// multiple of the SM count (persistent grid-stride loops).
#include <cuda_runtime.h>

#include <cmath>

#include "gemm_tc.cuh"
#include "host_util.h"
#include "internal.h"

namespace odl
{

namespace
{

constexpr int kSMs = 148;

inline int grid_for(int64_t work_items, int block, int per_sm = 8)
{
    int64_t blocks = (work_items + block - 1) / block;
    int64_t cap    = static_cast<int64_t>(kSMs) * per_sm;
    if (blocks > cap)
        blocks = cap;
    if (blocks < 1)
        blocks = 1;
    return static_cast<int>(blocks);
}

inline bool al16(const void *p)
{
    return (reinterpret_cast<uintptr_t>(p) & 15) == 0;
}

#define ODL_LAUNCH_CHECK(name)                                                      \
    ++::odl::g_launch_count;                                                        \
    do                                                                              \
    {                                                                               \
        cudaError_t _e = cudaGetLastError();                                        \
        if (_e != cudaSuccess)                                                      \
        {                                                                           \
            set_last_error(name " launch failed: %s", cudaGetErrorString(_e));      \
            return kCudaError;                                                      \
        }                                                                           \
    } while (0)

// ------------------------------------------------------------------------------------------------ ReLU
// y = x > 0 ? x : 0 ; optional low part of the TF32 split of y for a following 3xTF32 GEMM.
__global__ void relu_fwd_kernel(const float *__restrict__ x, float *__restrict__ y, float *__restrict__ y_small,
                                int64_t n, bool vec)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    int64_t i            = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (vec)
    {
        const int64_t n4 = n >> 2;
        for (; i < n4; i += stride)
        {
            float4 v = __ldg(reinterpret_cast<const float4 *>(x) + i);
            v.x = v.x > 0.f ? v.x : 0.f, v.y = v.y > 0.f ? v.y : 0.f, v.z = v.z > 0.f ? v.z : 0.f,
            v.w = v.w > 0.f ? v.w : 0.f;
            reinterpret_cast<float4 *>(y)[i] = v;
            if (y_small)
                reinterpret_cast<float4 *>(y_small)[i] =
                    make_float4(tf32_small(v.x), tf32_small(v.y), tf32_small(v.z), tf32_small(v.w));
        }
        i = (n4 << 2) + static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    }
    for (; i < n; i += stride)
    {
        float v = x[i];
        v       = v > 0.f ? v : 0.f;
        y[i]    = v;
        if (y_small)
            y_small[i] = tf32_small(v);
    }
}

// gx = gy * (ref > 0), ref being the forward input or output (same sign pattern).
__global__ void relu_bwd_kernel(const float *__restrict__ gy, const float *__restrict__ ref, float *__restrict__ gx,
                                int64_t n, bool vec)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    int64_t i            = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (vec)
    {
        const int64_t n4 = n >> 2;
        for (; i < n4; i += stride)
        {
            const float4 g = __ldg(reinterpret_cast<const float4 *>(gy) + i);
            const float4 r = __ldg(reinterpret_cast<const float4 *>(ref) + i);
            reinterpret_cast<float4 *>(gx)[i] =
                make_float4(r.x > 0.f ? g.x : 0.f, r.y > 0.f ? g.y : 0.f, r.z > 0.f ? g.z : 0.f, r.w > 0.f ? g.w : 0.f);
        }
        i = (n4 << 2) + static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    }
    for (; i < n; i += stride)
        gx[i] = ref[i] > 0.f ? gy[i] : 0.f;
}

// y[m,n] = x[m,n] + b[n]
__global__ void add_bias_kernel(const float *__restrict__ x, const float *__restrict__ b, float *__restrict__ y,
                                int64_t M, int64_t N)
{
    const int64_t total  = M * N;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride)
        y[i] = x[i] + __ldg(b + (i % N));
}

// ------------------------------------------------------------------------------------------------ softmax-CE
// a / b for many a and one b: q = a * (1/b) followed by one residual correction.  With a correctly rounded 1/b this
// yields the correctly rounded quotient (the value of a / b) except for rare operand pairs, where it is within one
// ulp, at a third of the instructions of a division.
__device__ __forceinline__ float div_by_common(float a, float b, float inv_b)
{
    const float q = a * inv_b;
    const float r = fmaf(-q, b, a);
    return fmaf(r, inv_b, q);
}

// One warp per row.  p = exp(x - max) / sum ; row_loss = log(p[t] + 1e-8) ; dlogits = (p - onehot) * scale.
// Rows of up to 32 * kSmCache classes are read from global memory ONCE and kept in registers (each exponential is
// computed once); longer rows fall back to re-reading.
constexpr int kSmCache = 32;
__global__ void __launch_bounds__(128) softmax_ce_kernel(const float *__restrict__ x, const int32_t *__restrict__ t32,
                                                         const int64_t *__restrict__ t64, int B, int C,
                                                         float *__restrict__ row_loss, float *__restrict__ dlogits,
                                                         float scale, int *__restrict__ err)
{
    const int lane = threadIdx.x & 31;
    const int row  = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (row >= B)
        return;
    const float *xr     = x + static_cast<int64_t>(row) * C;
    const int64_t label = t32 ? static_cast<int64_t>(t32[row]) : t64[row];
    if (label < 0 || label >= C)
    {
        if (lane == 0)
            if (err)
                atomicExch(err, 2);
        return;
    }
    const bool cached = C <= 32 * kSmCache;
    float v[kSmCache];
    float mx = -INFINITY;
    if (cached)
    {
#pragma unroll
        for (int i = 0; i < kSmCache; ++i)
        {
            const int c = lane + 32 * i;
            v[i]        = c < C ? xr[c] : -INFINITY;
            mx          = fmaxf(mx, v[i]);
        }
    }
    else
    {
        for (int c = lane; c < C; c += 32)
            mx = fmaxf(mx, xr[c]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
    if (cached)
    {
#pragma unroll
        for (int i = 0; i < kSmCache; ++i)
        {
            v[i] = (lane + 32 * i) < C ? expf(v[i] - mx) : 0.f;
            sum += v[i];
        }
    }
    else
    {
        for (int c = lane; c < C; c += 32)
            sum += expf(xr[c] - mx);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0 && row_loss)
    {
        const float pt = expf(xr[label] - mx) / sum;
        row_loss[row]  = logf(pt + 1e-8f);
    }
    if (dlogits)
    {
        float *dr       = dlogits + static_cast<int64_t>(row) * C;
        const float inv = 1.0f / sum;
        if (cached)
        {
#pragma unroll
            for (int i = 0; i < kSmCache; ++i)
            {
                const int c = lane + 32 * i;
                if (c < C)
                    dr[c] = (div_by_common(v[i], sum, inv) - (c == label ? 1.0f : 0.0f)) * scale;
            }
        }
        else
        {
            for (int c = lane; c < C; c += 32)
                dr[c] = (expf(xr[c] - mx) / sum - (c == label ? 1.0f : 0.0f)) * scale;
        }
    }
}

// loss = -(sum of row losses) / B, summed by one block in a fixed order (deterministic).
__global__ void __launch_bounds__(1024) loss_finalize_kernel(const float *__restrict__ row_loss, int B,
                                                             float *__restrict__ loss)
{
    __shared__ float red[1024];
    float s = 0.f;
    for (int i = threadIdx.x; i < B; i += 1024)
        s += row_loss[i];
    red[threadIdx.x] = s;
    __syncthreads();
    for (int o = 512; o > 0; o >>= 1)
    {
        if (threadIdx.x < o)
            red[threadIdx.x] += red[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0)
        loss[0] = -red[0] / static_cast<float>(B);
}

// ------------------------------------------------------------------------------------------------ optimizers
struct AdamArgs
{
    float b1, b2, one_m_b1, one_m_b2, mhat_scale, vhat_scale, eps, lr, hook_wd, grad_scale;
};

// Same operation order and per-operation fp32 rounding as the reference's chain of tensor ops (no contraction).
__device__ __forceinline__ float adam_one(float p, float &g, float &m, float &v, const AdamArgs &a)
{
    if (a.grad_scale != 1.0f)
        g = __fmul_rn(g, a.grad_scale);
    if (a.hook_wd > 0.0f)
        g = __fadd_rn(g, __fmul_rn(p, a.hook_wd));
    m               = __fadd_rn(__fmul_rn(m, a.b1), __fmul_rn(g, a.one_m_b1));
    v               = __fadd_rn(__fmul_rn(v, a.b2), __fmul_rn(__fmul_rn(g, g), a.one_m_b2));
    const float mh  = __fmul_rn(m, a.mhat_scale);
    const float vh  = __fmul_rn(v, a.vhat_scale);
    const float den = __fadd_rn(__fsqrt_rn(vh), a.eps);  // the reference's powf(vh, 0.5f)
    const float upd = __fdiv_rn(mh, den);
    return __fsub_rn(p, __fmul_rn(upd, a.lr));
}

__global__ void adam_kernel(float *__restrict__ p, float *__restrict__ g, float *__restrict__ m, float *__restrict__ v,
                            float *__restrict__ p_small, int64_t n, AdamArgs a, bool vec)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    int64_t i            = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const bool write_g   = (a.hook_wd > 0.0f) || (a.grad_scale != 1.0f);
    if (vec)
    {
        const int64_t n4 = n >> 2;
        for (; i < n4; i += stride)
        {
            float4 P = reinterpret_cast<float4 *>(p)[i], G = reinterpret_cast<float4 *>(g)[i];
            float4 Mv = reinterpret_cast<float4 *>(m)[i], V = reinterpret_cast<float4 *>(v)[i];
            P.x = adam_one(P.x, G.x, Mv.x, V.x, a);
            P.y = adam_one(P.y, G.y, Mv.y, V.y, a);
            P.z = adam_one(P.z, G.z, Mv.z, V.z, a);
            P.w = adam_one(P.w, G.w, Mv.w, V.w, a);
            reinterpret_cast<float4 *>(p)[i] = P;
            reinterpret_cast<float4 *>(m)[i] = Mv;
            reinterpret_cast<float4 *>(v)[i] = V;
            if (write_g)
                reinterpret_cast<float4 *>(g)[i] = G;
            if (p_small)
                reinterpret_cast<float4 *>(p_small)[i] =
                    make_float4(tf32_small(P.x), tf32_small(P.y), tf32_small(P.z), tf32_small(P.w));
        }
        i = (n4 << 2) + static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    }
    for (; i < n; i += stride)
    {
        float G = g[i], Mv = m[i], V = v[i];
        const float P = adam_one(p[i], G, Mv, V, a);
        p[i] = P, m[i] = Mv, v[i] = V;
        if (write_g)
            g[i] = G;
        if (p_small)
            p_small[i] = tf32_small(P);
    }
}

struct SgdArgs
{
    float lr, momentum, wd, hook_wd, grad_scale;
    int nesterov;
};

__device__ __forceinline__ float sgd_one(float p, float &g, float &buf, const SgdArgs &a)
{
    if (a.grad_scale != 1.0f)
        g = __fmul_rn(g, a.grad_scale);
    if (a.hook_wd > 0.0f)
        g = __fadd_rn(g, __fmul_rn(p, a.hook_wd));
    float gi = g;
    if (a.wd > 0.0f)
        gi = __fadd_rn(gi, __fmul_rn(p, a.wd));
    if (a.momentum > 0.0f)
    {
        buf = __fadd_rn(__fmul_rn(buf, a.momentum), gi);
        gi  = a.nesterov ? __fadd_rn(gi, __fmul_rn(buf, a.momentum)) : buf;
    }
    return __fsub_rn(p, __fmul_rn(gi, a.lr));
}

__global__ void sgd_kernel(float *__restrict__ p, float *__restrict__ g, float *__restrict__ buf,
                           float *__restrict__ p_small, int64_t n, SgdArgs a, bool vec)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    int64_t i            = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const bool write_g   = (a.hook_wd > 0.0f) || (a.grad_scale != 1.0f);
    const bool has_buf   = a.momentum > 0.0f;
    if (vec)
    {
        const int64_t n4 = n >> 2;
        for (; i < n4; i += stride)
        {
            float4 P = reinterpret_cast<float4 *>(p)[i], G = reinterpret_cast<float4 *>(g)[i];
            float4 Bf = has_buf ? reinterpret_cast<float4 *>(buf)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
            P.x = sgd_one(P.x, G.x, Bf.x, a);
            P.y = sgd_one(P.y, G.y, Bf.y, a);
            P.z = sgd_one(P.z, G.z, Bf.z, a);
            P.w = sgd_one(P.w, G.w, Bf.w, a);
            reinterpret_cast<float4 *>(p)[i] = P;
            if (has_buf)
                reinterpret_cast<float4 *>(buf)[i] = Bf;
            if (write_g)
                reinterpret_cast<float4 *>(g)[i] = G;
            if (p_small)
                reinterpret_cast<float4 *>(p_small)[i] =
                    make_float4(tf32_small(P.x), tf32_small(P.y), tf32_small(P.z), tf32_small(P.w));
        }
        i = (n4 << 2) + static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    }
    for (; i < n; i += stride)
    {
        float G = g[i], Bf = has_buf ? buf[i] : 0.f;
        const float P = sgd_one(p[i], G, Bf, a);
        p[i] = P;
        if (has_buf)
            buf[i] = Bf;
        if (write_g)
            g[i] = G;
        if (p_small)
            p_small[i] = tf32_small(P);
    }
}

// ------------------------------------------------------------------------------------------------ conv helpers
struct ConvGeom
{
    int N, C, H, W, KH, KW, S, P, OH, OW;
    int ckk;      // C*KH*KW
    int ld_col;   // ckk rounded up to a multiple of 4 (pad columns are written as zeros)
};

// col[(n*OH+oh)*OW+ow][(c*KH+kh)*KW+kw] = x[n,c,oh*S+kh-P,ow*S+kw-P] (0 outside); no padded image copy.
// One warp per output row: the (n, oh, ow) decomposition is done once per row, each lane owns groups of 4 consecutive
// columns (coalesced float4 stores) and decomposes its first column into (c, kh, kw) once, then steps kw / kh / c
// incrementally -- the kernel was bound by integer division, not by HBM, when every element did its own div/mod.
__global__ void __launch_bounds__(256) im2col_kernel(const float *__restrict__ x, float *__restrict__ col,
                                                     float *__restrict__ col_small, ConvGeom g, int64_t rows)
{
    const int q4          = g.ld_col >> 2;
    const int lane        = threadIdx.x & 31;
    const int64_t warp0   = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t n_warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
    const int khw         = g.KH * g.KW;
    for (int64_t row = warp0; row < rows; row += n_warps)
    {
        const int r32 = static_cast<int>(row);  // rows < 2^31 (checked by the launcher)
        const int ow  = r32 % g.OW;
        const int t   = r32 / g.OW;
        const int oh  = t % g.OH;
        const int n   = t / g.OH;
        const int h0 = oh * g.S - g.P, w0 = ow * g.S - g.P;
        const float *xn = x + static_cast<int64_t>(n) * g.C * g.H * g.W;
        for (int q = lane; q < q4; q += 32)
        {
            int cidx = q * 4;
            int c    = cidx / khw;
            int rem  = cidx - c * khw;
            int kh   = rem / g.KW;
            int kw   = rem - kh * g.KW;
            float v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
            {
                float val = 0.f;
                if (cidx + j < g.ckk)
                {
                    const int h = h0 + kh, w = w0 + kw;
                    if (h >= 0 && h < g.H && w >= 0 && w < g.W)
                        val = __ldg(xn + (static_cast<int64_t>(c) * g.H + h) * g.W + w);
                }
                v[j] = val;
                if (++kw == g.KW)
                {
                    kw = 0;
                    if (++kh == g.KH)
                    {
                        kh = 0;
                        ++c;
                    }
                }
            }
            const int64_t o = row * q4 + q;
            reinterpret_cast<float4 *>(col)[o] = make_float4(v[0], v[1], v[2], v[3]);
            if (col_small)
                reinterpret_cast<float4 *>(col_small)[o] =
                    make_float4(tf32_small(v[0]), tf32_small(v[1]), tf32_small(v[2]), tf32_small(v[3]));
        }
    }
}

// Flat NCHW index -> (n, c, h, w); 32-bit division whenever the index allows it (64-bit division is ~10x slower).
__device__ __forceinline__ void split_nchw_index(int64_t i, const ConvGeom &g, int &n, int &c, int &h, int &w)
{
    if (i <= 0x7fffffffLL)
    {
        unsigned u = static_cast<unsigned>(i);
        w          = static_cast<int>(u % static_cast<unsigned>(g.W));
        u /= static_cast<unsigned>(g.W);
        h = static_cast<int>(u % static_cast<unsigned>(g.H));
        u /= static_cast<unsigned>(g.H);
        c = static_cast<int>(u % static_cast<unsigned>(g.C));
        n = static_cast<int>(u / static_cast<unsigned>(g.C));
    }
    else
    {
        w         = static_cast<int>(i % g.W);
        int64_t t = i / g.W;
        h         = static_cast<int>(t % g.H);
        t /= g.H;
        c = static_cast<int>(t % g.C);
        n = static_cast<int>(t / g.C);
    }
}

// Gather form of col2im (no atomics): gx[n,c,h,w] = sum over (kh,kw) of colT[(c*KH+kh)*KW+kw][(n*OH+oh)*OW+ow]
// with oh = (h+P-kh)/S, ow = (w+P-kw)/S where those divide and are in range; (kh,kw) ascending like the reference's
// accumulation order.  colT is the TRANSPOSED column matrix [C*KH*KW][rows] so that a warp walking w reads
// consecutive addresses.
__global__ void col2im_gather_kernel(const float *__restrict__ colT, int64_t ld_colT, float *__restrict__ gx, ConvGeom g)
{
    const int64_t total  = static_cast<int64_t>(g.N) * g.C * g.H * g.W;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride)
    {
        int n, c, h, w;
        split_nchw_index(i, g, n, c, h, w);
        float acc = 0.f;
        // only taps with (h + P - kh) and (w + P - kw) divisible by the stride contribute: walk those directly
        const int hp = h + g.P, wp = w + g.P;
        const int kh0 = hp % g.S, kw0 = wp % g.S;
        const int ow0 = (wp - kw0) / g.S;
        int oh        = (hp - kh0) / g.S;
        for (int kh = kh0; kh < g.KH && oh >= 0; kh += g.S, --oh)
        {
            if (oh >= g.OH)
                continue;
            int ow = ow0;
            for (int kw = kw0; kw < g.KW && ow >= 0; kw += g.S, --ow)
            {
                if (ow >= g.OW)
                    continue;
                const int64_t r = (static_cast<int64_t>(n) * g.OH + oh) * g.OW + ow;
                acc += __ldg(colT + static_cast<int64_t>((c * g.KH + kh) * g.KW + kw) * ld_colT + r);
            }
        }
        gx[i] = acc;
    }
}

// Row-matrix col2im for the public im2col/col2im pair: same gather but reading col[rows][ld_col].
__global__ void col2im_rows_kernel(const float *__restrict__ col, float *__restrict__ gx, ConvGeom g)
{
    const int64_t total  = static_cast<int64_t>(g.N) * g.C * g.H * g.W;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride)
    {
        int n, c, h, w;
        split_nchw_index(i, g, n, c, h, w);
        float acc = 0.f;
        // only taps with (h + P - kh) and (w + P - kw) divisible by the stride contribute: walk those directly
        const int hp = h + g.P, wp = w + g.P;
        const int kh0 = hp % g.S, kw0 = wp % g.S;
        const int ow0 = (wp - kw0) / g.S;
        int oh        = (hp - kh0) / g.S;
        for (int kh = kh0; kh < g.KH && oh >= 0; kh += g.S, --oh)
        {
            if (oh >= g.OH)
                continue;
            int ow = ow0;
            for (int kw = kw0; kw < g.KW && ow >= 0; kw += g.S, --ow)
            {
                if (ow >= g.OW)
                    continue;
                const int64_t r = (static_cast<int64_t>(n) * g.OH + oh) * g.OW + ow;
                acc += __ldg(col + r * g.ld_col + (c * g.KH + kh) * g.KW + kw);
            }
        }
        gx[i] = acc;
    }
}

// gy[N][OC][HW] -> flat[N*HW][ld] (ld >= OC, pad columns zeroed) through a 32x33 shared tile; optional low part.
__global__ void __launch_bounds__(256) nchw_to_rows_kernel(const float *__restrict__ src, float *__restrict__ dst,
                                                           float *__restrict__ dst_small, int OC, int HW, int ld)
{
    __shared__ float tile[32][33];
    const int n   = blockIdx.z;
    const int hw0 = blockIdx.x * 32, oc0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
    for (int r = ty; r < 32; r += 8)
    {
        const int oc = oc0 + r, hw = hw0 + tx;
        tile[r][tx] = (oc < OC && hw < HW) ? __ldg(src + (static_cast<int64_t>(n) * OC + oc) * HW + hw) : 0.f;
    }
    __syncthreads();
    for (int r = ty; r < 32; r += 8)
    {
        const int hw = hw0 + r, oc = oc0 + tx;
        if (hw < HW && oc < ld)
        {
            const float v   = tile[tx][r];
            const int64_t o = (static_cast<int64_t>(n) * HW + hw) * ld + oc;
            dst[o]          = v;
            if (dst_small)
                dst_small[o] = tf32_small(v);
        }
    }
}

// gb[oc] = sum over n, hw of gy[n][oc][hw]: grid (OC, N, slabs of one plane); every block streams a contiguous piece
// of one (n, oc) plane (no per-element index arithmetic), reduces it and stores its partial sum at
// partial[(n * slabs + z) * OC + oc]; colsum_finish_launch then adds the partials of a channel in a fixed order.
__global__ void __launch_bounds__(256) channel_sum_kernel(const float *__restrict__ gy, float *__restrict__ partial, int OC,
                                                          int HW)
{
    __shared__ float red[256];
    const int oc = blockIdx.x, n = blockIdx.y;
    const float *plane = gy + (static_cast<int64_t>(n) * OC + oc) * HW;
    float s            = 0.f;
    for (int i = blockIdx.z * 256 + threadIdx.x; i < HW; i += gridDim.z * 256)
        s += __ldg(plane + i);
    red[threadIdx.x] = s;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1)
    {
        if (threadIdx.x < o)
            red[threadIdx.x] += red[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0)
        partial[(static_cast<size_t>(n) * gridDim.z + blockIdx.z) * OC + oc] = red[0];
}

}  // namespace

// ------------------------------------------------------------------------------------------------ launchers
int relu_forward_launch(const float *x, float *y, float *y_small, int64_t n, cudaStream_t s)
{
    if (!x || !y || n <= 0)
    {
        set_last_error("relu: invalid argument");
        return kInvalidArgument;
    }
    const bool vec = al16(x) && al16(y) && (!y_small || al16(y_small));
    relu_fwd_kernel<<<grid_for((n + 3) / 4, 256), 256, 0, s>>>(x, y, y_small, n, vec);
    ODL_LAUNCH_CHECK("relu_fwd_kernel");
    return kOk;
}

int relu_backward_launch(const float *gy, const float *ref, float *gx, int64_t n, cudaStream_t s)
{
    if (!gy || !ref || !gx || n <= 0)
    {
        set_last_error("relu_backward: invalid argument");
        return kInvalidArgument;
    }
    const bool vec = al16(gy) && al16(ref) && al16(gx);
    relu_bwd_kernel<<<grid_for((n + 3) / 4, 256), 256, 0, s>>>(gy, ref, gx, n, vec);
    ODL_LAUNCH_CHECK("relu_bwd_kernel");
    return kOk;
}

int add_bias_launch(const float *x, const float *b, float *y, int64_t M, int64_t N, cudaStream_t s)
{
    if (!x || !b || !y || M <= 0 || N <= 0)
    {
        set_last_error("add_bias: invalid argument");
        return kInvalidArgument;
    }
    add_bias_kernel<<<grid_for(M * N, 256), 256, 0, s>>>(x, b, y, M, N);
    ODL_LAUNCH_CHECK("add_bias_kernel");
    return kOk;
}

int softmax_ce_launch(const float *logits, const int32_t *t32, const int64_t *t64, int64_t B, int64_t C, float *loss,
                      float *dlogits, float *row_loss_scratch, float grad_scale, cudaStream_t s)
{
    if (!is_ready())
    {
        // the kernel reports an out-of-range label through the per-device flag odl_init allocates
        set_last_error("odl_init has not been called");
        return kNotInitialized;
    }
    if (!logits || (!t32 && !t64) || B <= 0 || C <= 0 || B > 0x7fffffff || C > 0x7fffffff)
    {
        set_last_error("softmax_ce: invalid argument (B=%lld C=%lld)", (long long)B, (long long)C);
        return kInvalidArgument;
    }
    if (loss && !row_loss_scratch)
    {
        set_last_error("softmax_ce: loss requested without row-loss scratch");
        return kInvalidArgument;
    }
    const float scale = grad_scale / static_cast<float>(B);
    softmax_ce_kernel<<<static_cast<int>((B + 3) / 4), 128, 0, s>>>(logits, t32, t64, (int)B, (int)C,
                                                                    loss ? row_loss_scratch : nullptr, dlogits, scale,
                                                                    device_error_flag());
    ODL_LAUNCH_CHECK("softmax_ce_kernel");
    if (loss)
    {
        loss_finalize_kernel<<<1, 1024, 0, s>>>(row_loss_scratch, (int)B, loss);
        ODL_LAUNCH_CHECK("loss_finalize_kernel");
    }
    return kOk;
}

int adam_launch(float *p, float *g, float *m, float *v, float *p_small, int64_t n, int t, float lr, float b1, float b2,
                float eps, float hook_wd, float grad_scale, cudaStream_t s)
{
    if (!p || !g || !m || !v || n <= 0 || t < 1)
    {
        set_last_error("adam: invalid argument (n=%lld t=%d)", (long long)n, t);
        return kInvalidArgument;
    }
    AdamArgs a;
    a.b1 = b1, a.b2 = b2;
    a.one_m_b1 = 1.0f - b1, a.one_m_b2 = 1.0f - b2;
    // bias corrections exactly as the reference computes them on the host (float pow, float reciprocal)
    const float b1p = std::pow(b1, static_cast<float>(t)), b2p = std::pow(b2, static_cast<float>(t));
    a.mhat_scale = 1.0f / (1.0f - b1p), a.vhat_scale = 1.0f / (1.0f - b2p);
    a.eps = eps, a.lr = lr, a.hook_wd = hook_wd, a.grad_scale = grad_scale;
    const bool vec = al16(p) && al16(g) && al16(m) && al16(v) && (!p_small || al16(p_small));
    adam_kernel<<<grid_for((n + 3) / 4, 256), 256, 0, s>>>(p, g, m, v, p_small, n, a, vec);
    ODL_LAUNCH_CHECK("adam_kernel");
    return kOk;
}

int sgd_launch(float *p, float *g, float *buf, float *p_small, int64_t n, float lr, float momentum, float wd,
               int nesterov, float hook_wd, float grad_scale, cudaStream_t s)
{
    if (!p || !g || n <= 0 || (momentum > 0.0f && !buf))
    {
        set_last_error("sgd: invalid argument (n=%lld)", (long long)n);
        return kInvalidArgument;
    }
    SgdArgs a{lr, momentum, wd, hook_wd, grad_scale, nesterov};
    const bool vec = al16(p) && al16(g) && (!buf || al16(buf)) && (!p_small || al16(p_small));
    sgd_kernel<<<grid_for((n + 3) / 4, 256), 256, 0, s>>>(p, g, buf, p_small, n, a, vec);
    ODL_LAUNCH_CHECK("sgd_kernel");
    return kOk;
}

namespace
{
int make_geom(int64_t N, int64_t C, int64_t H, int64_t W, int KH, int KW, int S, int P, ConvGeom *g)
{
    if (N <= 0 || C <= 0 || H <= 0 || W <= 0 || KH <= 0 || KW <= 0 || S <= 0 || P < 0 || N > 65535)
    {
        set_last_error("conv: invalid geometry");
        return kInvalidArgument;
    }
    const int OH = (int)((H + 2 * P - KH) / S + 1), OW = (int)((W + 2 * P - KW) / S + 1);
    if (OH <= 0 || OW <= 0)
    {
        set_last_error("conv2d: invalid output size OH=%d, OW=%d", OH, OW);
        return kInvalidArgument;
    }
    g->N = (int)N, g->C = (int)C, g->H = (int)H, g->W = (int)W, g->KH = KH, g->KW = KW, g->S = S, g->P = P;
    g->OH = OH, g->OW = OW;
    g->ckk    = (int)(C * KH * KW);
    g->ld_col = (g->ckk + 3) & ~3;
    return kOk;
}
}  // namespace

int conv_out_size(int64_t in, int k, int s, int p)
{
    return (int)((in + 2 * p - k) / s + 1);
}

int im2col_launch(const float *x, float *col, float *col_small, int64_t N, int64_t C, int64_t H, int64_t W, int KH, int KW,
                  int S, int P, cudaStream_t s)
{
    ConvGeom g;
    int rc = make_geom(N, C, H, W, KH, KW, S, P, &g);
    if (rc)
        return rc;
    if (!x || !col || !al16(col) || (col_small && !al16(col_small)))
    {
        set_last_error("im2col: null or misaligned buffer");
        return kInvalidArgument;
    }
    const int64_t rows = static_cast<int64_t>(g.N) * g.OH * g.OW;
    if (rows > 0x7fffffff)
    {
        set_last_error("im2col: more than 2^31-1 output rows");
        return kTooLarge;
    }
    im2col_kernel<<<grid_for(rows * 32, 256, 16), 256, 0, s>>>(x, col, col_small, g, rows);
    ODL_LAUNCH_CHECK("im2col_kernel");
    return kOk;
}

int col2im_launch(const float *col, int transposed, int64_t ld, float *gx, int64_t N, int64_t C, int64_t H, int64_t W,
                  int KH, int KW, int S, int P, cudaStream_t s)
{
    ConvGeom g;
    int rc = make_geom(N, C, H, W, KH, KW, S, P, &g);
    if (rc)
        return rc;
    if (!col || !gx)
    {
        set_last_error("col2im: null buffer");
        return kInvalidArgument;
    }
    const int64_t total = N * C * H * W;
    if (transposed)
    {
        col2im_gather_kernel<<<grid_for(total, 256, 16), 256, 0, s>>>(col, ld, gx, g);
    }
    else
    {
        g.ld_col = (int)ld;
        col2im_rows_kernel<<<grid_for(total, 256, 16), 256, 0, s>>>(col, gx, g);
    }
    ODL_LAUNCH_CHECK("col2im kernel");
    return kOk;
}

int nchw_to_rows_launch(const float *src, float *dst, float *dst_small, int64_t N, int64_t OC, int64_t HW, int64_t ld,
                        cudaStream_t s)
{
    dim3 grid((unsigned)((HW + 31) / 32), (unsigned)((ld + 31) / 32), (unsigned)N);
    nchw_to_rows_kernel<<<grid, 256, 0, s>>>(src, dst, dst_small, (int)OC, (int)HW, (int)ld);
    ODL_LAUNCH_CHECK("nchw_to_rows_kernel");
    return kOk;
}

int channel_sum_launch(const float *gy, float *gb, int64_t N, int64_t OC, int64_t HW, cudaStream_t s)
{
    if (N > 65535 || OC > 0x7fffffff || HW > 0x7fffffff)
    {
        set_last_error("channel_sum: dimension out of range");
        return kTooLarge;
    }
    ODL_CUDA_TRY(cudaMemsetAsync(gb, 0, OC * sizeof(float), s));
    int slabs = (int)((HW + 256 * 16 - 1) / (256 * 16));
    if (slabs > 64)
        slabs = 64;
    dim3 grid((unsigned)OC, (unsigned)N, (unsigned)slabs);
    float *partial = colsum_partial_scratch((int)(N * slabs), OC);
    if (!partial)
        return kCudaError;
    channel_sum_kernel<<<grid, 256, 0, s>>>(gy, partial, (int)OC, (int)HW);
    ODL_LAUNCH_CHECK("channel_sum_kernel");
    return colsum_finish_launch(partial, (int)(N * slabs), OC, (int)OC, gb, s);
}

}  // namespace odl
