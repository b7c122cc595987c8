// extern "C" layer: library state (device binding, error flag, scratch arena) and the GEMM entry points.
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "../../include/odl_b200.h"
#include "gemm_tc.cuh"
#include "host_util.h"
#include "internal.h"

namespace odl
{

namespace
{
thread_local char g_err[1024] = {0};

struct DeviceState
{
    bool ready      = false;
    int device      = -1;
    int *err_flag   = nullptr;  // device memory
    char *arena     = nullptr;
    size_t capacity = 0;
    size_t used     = 0;
};
DeviceState g_state;
std::mutex g_mu;
long long g_scratch_generation = 0;
}  // namespace

// Library-owned scratch blocks (the arena below, the column-sum scratch of split.cu) are replaced when a call needs
// more than they hold.  Every replacement bumps this counter, so that whoever recorded raw scratch addresses (a CUDA
// graph of the training step) can tell that they are stale.
long long scratch_generation()
{
    return g_scratch_generation;
}

void bump_scratch_generation()
{
    ++g_scratch_generation;
}

void set_last_error(const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

const char *get_last_error()
{
    return g_err;
}

int *device_error_flag()
{
    return g_state.err_flag;
}

bool is_ready()
{
    return g_state.ready;
}

void arena_reset()
{
    g_state.used = 0;
}

// Bump allocation out of one device block.  Growing replaces the block: work already queued may still read the
// old one, so the device is drained first (this happens a handful of times while sizes warm up, never in steady state).
void *arena_alloc(size_t bytes)
{
    bytes = (bytes + 255) & ~size_t(255);
    if (g_state.used + bytes > g_state.capacity)
    {
        if (g_state.used != 0)
        {
            // A call needs more than the block holds and already carved part of it: the caller sizes the
            // whole call up front with arena_reserve, so reaching this is a programming error.
            set_last_error("scratch arena: reserve(%zu) was not called before alloc", g_state.used + bytes);
            return nullptr;
        }
        if (cudaDeviceSynchronize() != cudaSuccess)
            return nullptr;
        if (g_state.arena)
            cudaFree(g_state.arena);
        g_state.arena    = nullptr;
        g_state.capacity = 0;
        size_t want      = bytes + (bytes >> 2);
        void *p          = nullptr;
        cudaError_t e    = cudaMalloc(&p, want);
        if (e != cudaSuccess)
        {
            set_last_error("scratch arena: cudaMalloc(%zu) failed: %s", want, cudaGetErrorString(e));
            return nullptr;
        }
        g_state.arena    = static_cast<char *>(p);
        g_state.capacity = want;
        bump_scratch_generation();
    }
    void *out = g_state.arena + g_state.used;
    g_state.used += bytes;
    return out;
}

// Make sure one call's total scratch fits; must be called right after arena_reset().
int arena_reserve(size_t total_bytes)
{
    total_bytes += 4096;
    if (total_bytes <= g_state.capacity)
        return kOk;
    void *p = arena_alloc(total_bytes);
    if (!p)
        return kCudaError;
    g_state.used = 0;
    return kOk;
}

namespace
{
inline bool misaligned(const void *p, int64_t ld)
{
    return (reinterpret_cast<uintptr_t>(p) & 15) || (ld & 3);
}
inline int64_t pad4(int64_t x)
{
    return (x + 3) & ~int64_t(3);
}
inline size_t a256(size_t x)
{
    return (x + 255) & ~size_t(255);
}

struct Prepared
{
    const float *big;
    const float *small;
    int64_t ld;
};

size_t operand_scratch_impl(const float *ptr, const float *small, int64_t ld, int64_t rows, int64_t cols, int terms)
{
    if (misaligned(ptr, ld))
        return a256(rows * pad4(cols) * 4) * (terms == 3 ? 2 : 1);
    if (terms == 3 && (!small || misaligned(small, ld)))
        return a256(rows * ld * 4);
    return 0;
}

int prepare_operand(const float *ptr, const float *small, int64_t ld, int64_t rows, int64_t cols, int terms,
                    cudaStream_t stream, Prepared *out)
{
    if (misaligned(ptr, ld))
    {
        const int64_t ldp = pad4(cols);
        float *big        = static_cast<float *>(arena_alloc(rows * ldp * 4));
        float *sm         = terms == 3 ? static_cast<float *>(arena_alloc(rows * ldp * 4)) : nullptr;
        if (!big || (terms == 3 && !sm))
            return kCudaError;
        int rc = split_launch(ptr, ld, (int)rows, (int)cols, nullptr, 0, big, sm, ldp, nullptr, stream);
        if (rc)
            return rc;
        *out = Prepared{big, sm, ldp};
        return kOk;
    }
    if (terms == 3 && (!small || misaligned(small, ld)))
    {
        float *sm = static_cast<float *>(arena_alloc(rows * ld * 4));
        if (!sm)
            return kCudaError;
        int rc = split_launch(ptr, ld, (int)rows, (int)cols, nullptr, 0, nullptr, sm, ld, nullptr, stream);
        if (rc)
            return rc;
        *out = Prepared{ptr, sm, ld};
        return kOk;
    }
    *out = Prepared{ptr, small, ld};
    return kOk;
}
}  // namespace

// Scratch bytes gemm_dispatch will carve for one operand (padded copy and/or low part).
size_t operand_scratch(const float *ptr, const float *small, int64_t ld, int64_t rows, int64_t cols, int terms)
{
    return operand_scratch_impl(ptr, small, ld, rows, cols, terms);
}

// The GEMM every fused entry point funnels into.  `reset_arena` is false when the caller already carved scratch
// for this call (Linear / conv orchestration) and reserved enough for the operand splits too.
int gemm_dispatch(int transA, int transB, int64_t M, int64_t N, int64_t K, const float *A, const float *A_small,
                  int64_t lda, const float *B, const float *B_small, int64_t ldb, float *D, float *D_small, int64_t ldd,
                  const float *bias, const float *mask_src, int64_t ld_mask, float *colsum, int flags, int precision,
                  cudaStream_t stream, bool reset_arena, int ohw, const float *scale)
{
    if (!is_ready())
    {
        set_last_error("odl_init has not been called");
        return kNotInitialized;
    }
    if (M <= 0 || N <= 0 || K <= 0 || !A || !B || !D)
    {
        set_last_error("gemm: invalid argument (M=%lld N=%lld K=%lld A=%p B=%p D=%p)", (long long)M, (long long)N,
                       (long long)K, (const void *)A, (const void *)B, (void *)D);
        return kInvalidArgument;
    }
    if (M > 0x7fffffff || N > 0x7fffffff || K > 0x7fffffff)
    {
        set_last_error("gemm: dimension exceeds 2^31-1");
        return kTooLarge;
    }
    if (precision != ODL_PRECISION_3XTF32 && precision != ODL_PRECISION_TF32)
    {
        set_last_error("gemm: unknown precision %d", precision);
        return kInvalidArgument;
    }
    if (((flags & kEpiBias) && !bias) || ((flags & kEpiMask) && !mask_src) || ((flags & kEpiColsum) && !colsum) ||
        ((flags & kEpiSmall) && !D_small) || ((flags & kEpiScale) && !scale) ||
        ((flags & (kEpiScale | kEpiSilu)) && !(flags & kEpiNCHW)))
    {
        set_last_error("gemm: epilogue flag 0x%x set without its pointer", flags);
        return kInvalidArgument;
    }
    const int terms      = precision == ODL_PRECISION_3XTF32 ? 3 : 1;
    const int64_t a_rows = transA ? K : M, a_cols = transA ? M : K;
    const int64_t b_rows = transB ? N : K, b_cols = transB ? K : N;
    if (lda < a_cols || ldb < b_cols || ldd < N)
    {
        set_last_error("gemm: leading dimension smaller than the row length (lda=%lld ldb=%lld ldd=%lld)",
                       (long long)lda, (long long)ldb, (long long)ldd);
        return kInvalidArgument;
    }
    if (reset_arena)
    {
        arena_reset();
        int rc = arena_reserve(operand_scratch_impl(A, A_small, lda, a_rows, a_cols, terms) +
                               operand_scratch_impl(B, B_small, ldb, b_rows, b_cols, terms));
        if (rc)
            return rc;
    }
    Prepared pa, pb;
    int rc;
    if ((rc = prepare_operand(A, A_small, lda, a_rows, a_cols, terms, stream, &pa)))
        return rc;
    if ((rc = prepare_operand(B, B_small, ldb, b_rows, b_cols, terms, stream, &pb)))
        return rc;
    GemmParams p;
    p.D       = D;
    p.D_small = D_small;
    p.bias    = bias;
    p.scale   = scale;
    p.aux     = mask_src;
    p.colsum    = nullptr;
    p.ld_colsum = 0;
    const int slabs = static_cast<int>((M + 127) / 128) * 4;  // 32-row slabs of whole 128-row tiles
    if (flags & kEpiColsum)
    {
        p.ld_colsum = static_cast<int>(pad4(N));
        p.colsum    = colsum_partial_scratch(slabs, p.ld_colsum);
        if (!p.colsum)
            return kCudaError;
    }
    p.err     = device_error_flag();
    p.M       = (int)M;
    p.N       = (int)N;
    p.K       = (int)K;
    p.ldd     = (int)ldd;
    p.ld_aux  = (int)ld_mask;
    p.flags   = flags;
    p.ohw     = ohw;
    p.kb_per_split = 0;
    const int a_mn = transA ? 1 : 0;
    const int b_mn = transB ? 0 : 1;
    rc = gemm_tc_launch(pa.big, pa.small, pa.ld, a_mn, pb.big, pb.small, pb.ld, b_mn, p, terms, g_bn_override, stream);
    if (rc == kOk && (flags & kEpiColsum))
        rc = colsum_finish_launch(p.colsum, slabs, p.ld_colsum, (int)N, colsum, stream);
    return rc;
}

int g_bn_override = 0;
long long g_launch_count = 0;

}  // namespace odl

using namespace odl;

extern "C" {

int odl_init(int device)
{
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_state.ready && g_state.device == device)
        return kOk;
    if (g_state.ready)
    {
        set_last_error("odl_init: already bound to device %d (one device per process)", g_state.device);
        return kInvalidArgument;
    }
    ODL_CUDA_TRY(cudaSetDevice(device));
    cudaDeviceProp prop;
    ODL_CUDA_TRY(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
    {
        set_last_error("odl_init: device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major,
                       prop.minor);
        return kCudaError;
    }
    ODL_CUDA_TRY(cudaMalloc(&g_state.err_flag, sizeof(int)));
    ODL_CUDA_TRY(cudaMemset(g_state.err_flag, 0, sizeof(int)));
    g_state.device = device;
    g_state.ready  = true;
    return kOk;
}

const char *odl_last_error(void)
{
    return get_last_error();
}

int odl_device_status(void *stream)
{
    if (!is_ready())
    {
        set_last_error("odl_init has not been called");
        return kNotInitialized;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int flag       = 0;
    ODL_CUDA_TRY(cudaMemcpyAsync(&flag, g_state.err_flag, sizeof(int), cudaMemcpyDeviceToHost, s));
    ODL_CUDA_TRY(cudaStreamSynchronize(s));
    if (flag != 0)
    {
        ODL_CUDA_TRY(cudaMemsetAsync(g_state.err_flag, 0, sizeof(int), s));
        ODL_CUDA_TRY(cudaStreamSynchronize(s));
        if (flag == 2)
        {
            set_last_error("softmax_cross_entropy: label out of range");
            return kInvalidArgument;
        }
        if (flag == 3)
        {
            set_last_error("gather_rows: sample index out of range");
            return kInvalidArgument;
        }
        gemm_pair_recover(s);  // a persistent GEMM that gave up may have left its unit counters mid-launch
        ODL_CUDA_TRY(cudaStreamSynchronize(s));
        set_last_error("a kernel gave up on a bounded wait (pipeline barrier never completed)");
        return kKernelTimeout;
    }
    return kOk;
}

int64_t odl_scratch_bytes(void)
{
    return static_cast<int64_t>(g_state.capacity);
}

long long odl_scratch_generation(void)
{
    return scratch_generation();
}

int odl_debug_set_split_k(int splits)
{
    g_split_k = splits;
    return kOk;
}

// Test hook: K-blocks of 32 accumulated in TMEM between drains into registers (0 = default).
int odl_debug_set_chunk(int chunk_kb)
{
    g_chunk_kb = chunk_kb;
    return kOk;
}

// Test hook: force the GEMM column-tile width (64, 128, 256; 0 = automatic).
int odl_debug_set_tile_n(int bn)
{
    g_bn_override = bn;
    return kOk;
}

int odl_gemm_ex(int transA, int transB, int64_t M, int64_t N, int64_t K, const float *A, const float *A_small,
                int64_t lda, const float *B, const float *B_small, int64_t ldb, float *D, float *D_small, int64_t ldd,
                const float *bias, const float *mask_src, int64_t ld_mask, float *colsum, int epilogue_flags,
                int precision, void *stream)
{
    return gemm_dispatch(transA, transB, M, N, K, A, A_small, lda, B, B_small, ldb, D, D_small, ldd, bias, mask_src,
                         ld_mask, colsum, epilogue_flags, precision, static_cast<cudaStream_t>(stream), true);
}

int odl_matmul(const float *A, const float *B, float *C, int64_t M, int64_t N, int64_t K, int64_t batch, int b_batched,
               int precision, void *stream)
{
    if (batch < 1)
    {
        set_last_error("matmul: batch must be >= 1");
        return kInvalidArgument;
    }
    if (batch > 1 && !b_batched)
    {
        // [batch, M, K] x [K, N] is one GEMM over batch*M rows
        return gemm_dispatch(0, 0, batch * M, N, K, A, nullptr, K, B, nullptr, N, C, nullptr, N, nullptr, nullptr, 0,
                             nullptr, 0, precision, static_cast<cudaStream_t>(stream), true);
    }
    for (int64_t i = 0; i < batch; ++i)
    {
        int rc = gemm_dispatch(0, 0, M, N, K, A + i * M * K, nullptr, K, B + i * K * N, nullptr, N, C + i * M * N,
                               nullptr, N, nullptr, nullptr, 0, nullptr, 0, precision,
                               static_cast<cudaStream_t>(stream), true);
        if (rc)
            return rc;
    }
    return kOk;
}

int odl_split_tf32(const float *src, int64_t ld_src, int64_t rows, int64_t cols, const float *mask_src, int64_t ld_mask,
                   float *dst_big, float *dst_small, int64_t ld_dst, float *colsum, void *stream)
{
    if (rows > 0x7fffffff || cols > 0x7fffffff)
    {
        set_last_error("split: dimension exceeds 2^31-1");
        return kTooLarge;
    }
    return split_launch(src, ld_src, (int)rows, (int)cols, mask_src, ld_mask, dst_big, dst_small, ld_dst, colsum,
                        static_cast<cudaStream_t>(stream));
}


#define ST(x) static_cast<cudaStream_t>(x)

int odl_linear_forward(const float *x, const float *x_small, const float *w, const float *w_small, const float *b,
                       float *y, float *y_small, int64_t M, int64_t N, int64_t K, int w_layout, int relu, int precision,
                       void *stream)
{
    return linear_forward(x, x_small, w, w_small, b, y, y_small, M, N, K, w_layout, relu, precision, ST(stream));
}

int odl_linear_backward(const float *x, const float *x_small, const float *w, const float *w_small, const float *dy,
                        const float *y, float *dx, float *dw, float *db, int64_t M, int64_t N, int64_t K, int w_layout,
                        int precision, void *stream)
{
    return linear_backward(x, x_small, w, w_small, dy, nullptr, y, dx, nullptr, nullptr, nullptr, dw, db, M, N, K, w_layout,
                           precision, ST(stream));
}

int odl_linear_backward_chain(const float *x, const float *x_small, const float *w, const float *w_small, const float *dy, const float *dy_small,
                              const float *y, float *dx, float *dx_small, const float *prev_y, float *prev_db, float *dw,
                              float *db, int64_t M, int64_t N, int64_t K, int w_layout, int precision, void *stream)
{
    return linear_backward(x, x_small, w, w_small, dy, dy_small, y, dx, dx_small, prev_y, prev_db, dw, db, M, N, K, w_layout,
                           precision, ST(stream));
}

int odl_relu_forward(const float *x, float *y, int64_t n, void *stream)
{
    return relu_forward_launch(x, y, nullptr, n, ST(stream));
}

int odl_relu_backward(const float *gy, const float *x_or_y, float *gx, int64_t n, void *stream)
{
    return relu_backward_launch(gy, x_or_y, gx, n, ST(stream));
}

int odl_add_bias(const float *x, const float *b, float *y, int64_t M, int64_t N, void *stream)
{
    return add_bias_launch(x, b, y, M, N, ST(stream));
}

int odl_sum_to_row(const float *g, float *out, int64_t M, int64_t N, void *stream)
{
    if (!g || !out || M <= 0 || N <= 0 || M > 0x7fffffff || N > 0x7fffffff)
    {
        set_last_error("sum_to_row: invalid argument");
        return kInvalidArgument;
    }
    ODL_CUDA_TRY(cudaMemsetAsync(out, 0, static_cast<size_t>(N) * 4, ST(stream)));
    return split_launch(g, N, (int)M, (int)N, nullptr, 0, nullptr, nullptr, N, out, ST(stream));
}

int odl_softmax_cross_entropy(const float *logits, const void *labels, int labels_are_int64, int64_t B, int64_t C,
                              float *loss, float *dlogits, float grad_scale, void *stream)
{
    if (!is_ready())
    {
        set_last_error("odl_init has not been called");
        return kNotInitialized;
    }
    float *rows = nullptr;
    if (loss)
    {
        arena_reset();
        int rc = arena_reserve(static_cast<size_t>(B) * 4 + 256);
        if (rc)
            return rc;
        rows = static_cast<float *>(arena_alloc(static_cast<size_t>(B) * 4));
        if (!rows)
            return kCudaError;
    }
    return softmax_ce_launch(logits, labels_are_int64 ? nullptr : static_cast<const int32_t *>(labels),
                             labels_are_int64 ? static_cast<const int64_t *>(labels) : nullptr, B, C, loss, dlogits, rows,
                             grad_scale, ST(stream));
}

int odl_adam_step(float *param, float *grad, float *m, float *v, float *param_small, int64_t n, int t, float lr,
                  float beta1, float beta2, float eps, float hook_weight_decay, float grad_scale, void *stream)
{
    return adam_launch(param, grad, m, v, param_small, n, t, lr, beta1, beta2, eps, hook_weight_decay, grad_scale,
                       ST(stream));
}

int odl_sgd_step(float *param, float *grad, float *momentum_buf, float *param_small, int64_t n, float lr, float momentum,
                 float weight_decay, int nesterov, float hook_weight_decay, float grad_scale, void *stream)
{
    return sgd_launch(param, grad, momentum_buf, param_small, n, lr, momentum, weight_decay, nesterov, hook_weight_decay,
                      grad_scale, ST(stream));
}

int odl_im2col(const float *x, float *col, int64_t N, int64_t C, int64_t H, int64_t W, int KH, int KW, int stride, int pad,
               void *stream)
{
    // the public form writes rows of exactly C*KH*KW columns, like the reference
    if ((C * KH * KW) & 3)
    {
        set_last_error("im2col: C*KH*KW must be a multiple of 4 for the row-matrix form (got %lld)",
                       (long long)(C * KH * KW));
        return kInvalidArgument;
    }
    return im2col_launch(x, col, nullptr, N, C, H, W, KH, KW, stride, pad, ST(stream));
}

int odl_col2im(const float *col, float *x, int64_t N, int64_t C, int64_t H, int64_t W, int KH, int KW, int stride, int pad,
               void *stream)
{
    return col2im_launch(col, 0, C * KH * KW, x, N, C, H, W, KH, KW, stride, pad, ST(stream));
}

int odl_conv2d_forward(const float *x, const float *w, const float *b, float *y, int64_t N, int64_t C, int64_t H,
                       int64_t W, int64_t OC, int KH, int KW, int stride, int pad, int relu, int precision, void *stream)
{
    return conv2d_forward(x, w, b, y, N, C, H, W, OC, KH, KW, stride, pad, relu, precision, ST(stream));
}

int odl_conv2d_bn_act_forward(const float *x, const float *w, const float *scale, const float *shift, float *y, int64_t N,
                              int64_t C, int64_t H, int64_t W, int64_t OC, int KH, int KW, int stride, int pad, int act,
                              int precision, void *stream)
{
    if (!scale || !shift)
    {
        set_last_error("conv2d_bn_act_forward: scale and shift are required (see odl_batch_norm_fold)");
        return kInvalidArgument;
    }
    return conv2d_forward(x, w, shift, y, N, C, H, W, OC, KH, KW, stride, pad, act, precision, ST(stream), scale);
}

int odl_conv2d_backward(const float *gy, const float *x, const float *w, float *gx, float *gw, float *gb, int64_t N,
                        int64_t C, int64_t H, int64_t W, int64_t OC, int KH, int KW, int stride, int pad, int gy_layout,
                        int precision, void *stream)
{
    return conv2d_backward(gy, x, w, gx, gw, gb, N, C, H, W, OC, KH, KW, stride, pad, gy_layout, precision, ST(stream));
}

}  // extern "C"

extern "C" long long odl_launch_count(void)
{
    return odl::g_launch_count;
}

namespace odl
{
extern int g_bk_override;
}
// Test hook: K elements per pipeline stage of the 256-wide GEMM tile (16 or 32; 0 = automatic).
extern "C" int odl_debug_set_bk(int bk)
{
    odl::g_bk_override = bk;
    return 0;
}

namespace odl
{
extern int g_slabs;
}
// Test hook: K-slabs per pipeline stage of the 1-CTA kernel in plain TF32 (0 = automatic, 1 or 2).
extern "C" int odl_debug_set_slabs(int n)
{
    odl::g_slabs = n;
    return 0;
}

// Test hook: CTA pairs the persistent GEMM kernel walks its tiles with (0 = as many as the GPU holds at once).
extern "C" int odl_debug_set_persistent_pairs(int pairs)
{
    odl::g_persist_pairs = pairs;
    return 0;
}

// Test hook: 0 = stream-K in the persistent GEMM where it pays, 1 = always, -1 = never.
extern "C" int odl_debug_set_stream_k(int mode)
{
    odl::g_stream_k = mode;
    return 0;
}

// Test hook: device address of the per-device error flag (NULL before odl_init), for test kernels that raise it the way
// a timed-out GEMM does.
extern "C" int *odl_debug_error_flag(void)
{
    return odl::device_error_flag();
}

// Test hook: 0 = pair (2-CTA) GEMM kernel where it pays, 1 = never, 2 = whenever the shape allows it.
extern "C" int odl_debug_set_pair_mode(int mode)
{
    odl::g_pair_mode = mode;
    return 0;
}
