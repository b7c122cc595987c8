/*
 * TEST INFRASTRUCTURE -- not product code.  Nothing outside tests/, __graft_entry__.smoke() and the
 * cpu_baseline / reference legs of bench.py may load this file's library.
 *
 * Plain-C restatement of the OriginDL reference's CPU arithmetic for the dense hot path: same loops, same
 * single fp32 accumulators, same operation order, so that results agree with the reference's CPU backend to
 * the last bit wherever the compiler does not contract a*b+c (built with -ffp-contract=off; the reference is
 * built -O2 for x86-64 without FMA, so neither side contracts).
 *
 * Parity is PINNED: tests/test_oracle_vs_reference.py checks every function here against the unmodified reference
 * library (oracle/_ref/libodl_ref.so, built by oracle/Makefile) on seeded inputs, and tests/test_oracle_golden.py
 * checks it against the known-answer vectors of the reference's own unit tests (tests/golden/).
 *
 * Each function names the reference source it follows (paths relative to the OriginDL tree).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* C[M,N] = A[M,K] . B[K,N]; one fp32 accumulator per output, k ascending.
 * src/mat/origin/cpu/math/matmul.cpp:26-41 (matmul_2d_impl). */
void oracle_matmul(const float *a, const float *b, float *c, int64_t M, int64_t N, int64_t K)
{
    for (int64_t i = 0; i < M; ++i)
        for (int64_t j = 0; j < N; ++j)
        {
            float sum = 0.0f;
            for (int64_t k = 0; k < K; ++k)
                sum += a[i * K + k] * b[k * N + j];
            c[i * N + j] = sum;
        }
}

/* out[C,R] = in[R,C]^T (materialised copy, as the reference's transpose()).
 * src/mat/origin/cpu/shape/transpose.cpp. */
void oracle_transpose(const float *in, float *out, int64_t R, int64_t C)
{
    for (int64_t r = 0; r < R; ++r)
        for (int64_t c = 0; c < C; ++c)
            out[c * R + r] = in[r * C + c];
}

/* db[n] = sum_m g[m,n], one accumulator, m ascending.
 * include/origin/mat/origin/device_common/operation_templates.h:269-340 (AxisSumCompute::axis_sum),
 * reached from BroadcastTo::backward -> sum_to (src/operators/math/broadcast_to.cpp:29-46). */
void oracle_colsum(const float *g, float *out, int64_t M, int64_t N)
{
    for (int64_t n = 0; n < N; ++n)
    {
        float s = 0.0f;
        for (int64_t m = 0; m < M; ++m)
            s += g[m * N + n];
        out[n] = s;
    }
}

/* y = relu(x . op(W) + b).  w_layout 0: W is [N,K] and op = transpose (functional::custom_linear,
 * src/operators/custom/linear.cpp:12-114, or mat_mul(x, transpose(W))); w_layout 1: W is [K,N] (nn::Linear,
 * src/nn/layers/linear.cpp:80-106).  Bias is added after the product (Add::forward, src/operators/math/add.cpp:12-27);
 * ReLU is value > 0 ? value : 0 (operation_templates.h:144-151).  b may be NULL; relu is a flag. */
void oracle_linear_forward(const float *x, const float *w, const float *b, float *y, int64_t M, int64_t N, int64_t K,
                           int w_layout, int relu)
{
    for (int64_t i = 0; i < M; ++i)
        for (int64_t j = 0; j < N; ++j)
        {
            float sum = 0.0f;
            if (w_layout == 0)
                for (int64_t k = 0; k < K; ++k)
                    sum += x[i * K + k] * w[j * K + k];
            else
                for (int64_t k = 0; k < K; ++k)
                    sum += x[i * K + k] * w[k * N + j];
            if (b)
                sum = sum + b[j];
            if (relu)
                sum = (sum > 0.0f) ? sum : 0.0f;
            y[i * N + j] = sum;
        }
}

/* Backward of the layer above for upstream gradient dy.
 *   g  = relu ? dy * (y > 0) : dy          ReLU::backward gx = gy * mask, mask = (x > 0) as 0/1 fp32
 *                                          (src/operators/activation/relu.cpp:23-54; y > 0 <=> pre-activation > 0)
 *   db = colsum(g)                         BroadcastTo::backward (src/operators/math/broadcast_to.cpp:29-46)
 *   dx = g . W ([N,K]) or g . W^T ([K,N])  MatMul::backward gx = gy . w^T (src/operators/math/mat_mul.cpp:171-177)
 *   dw = g^T . x ([N,K]) or x^T . g ([K,N])                 gw = x^T . gy
 * y is the forward OUTPUT (needed only when relu != 0).  dx, dw, db may each be NULL. */
void oracle_linear_backward(const float *x, const float *w, const float *y, const float *dy, float *dx, float *dw,
                            float *db, int64_t M, int64_t N, int64_t K, int w_layout, int relu)
{
    float *g = (float *)malloc(sizeof(float) * (size_t)M * (size_t)N);
    for (int64_t i = 0; i < M * N; ++i)
        g[i] = relu ? dy[i] * ((y[i] > 0.0f) ? 1.0f : 0.0f) : dy[i];
    if (db)
        oracle_colsum(g, db, M, N);
    if (dx)
        for (int64_t i = 0; i < M; ++i)
            for (int64_t k = 0; k < K; ++k)
            {
                float sum = 0.0f;
                if (w_layout == 0)
                    for (int64_t n = 0; n < N; ++n)
                        sum += g[i * N + n] * w[n * K + k];
                else
                    for (int64_t n = 0; n < N; ++n)
                        sum += g[i * N + n] * w[k * N + n];
                dx[i * K + k] = sum;
            }
    if (dw)
        for (int64_t n = 0; n < N; ++n)
            for (int64_t k = 0; k < K; ++k)
            {
                float sum = 0.0f;
                for (int64_t m = 0; m < M; ++m)
                    sum += x[m * K + k] * g[m * N + n];
                if (w_layout == 0)
                    dw[n * K + k] = sum;
                else
                    dw[k * N + n] = sum;
            }
    free(g);
}

/* p = softmax(x) row-wise with the row maximum subtracted.
 * src/operators/activation/softmax.cpp:14-76: max -> x - max -> exp -> sum (sequential) -> divide. */
static void softmax_rows(const float *x, float *p, int64_t B, int64_t C)
{
    for (int64_t i = 0; i < B; ++i)
    {
        float mx = x[i * C];
        for (int64_t c = 1; c < C; ++c)
            if (x[i * C + c] > mx)
                mx = x[i * C + c];
        float s = 0.0f;
        for (int64_t c = 0; c < C; ++c)
        {
            p[i * C + c] = expf(x[i * C + c] - mx);
            s += p[i * C + c];
        }
        for (int64_t c = 0; c < C; ++c)
            p[i * C + c] = p[i * C + c] / s;
    }
}

/* loss = -(1/B) * sum_i log(softmax(x)[i, t_i] + 1e-8);  dlogits = (softmax(x) - onehot(t)) * (1/B).
 * src/operators/loss/softmax_cross_entropy.cpp:17-75 (forward; the sum of logs is a sequential fp32 sum and the
 * division by B happens on the host in fp32) and :77-111 (backward with gy = 1: diff * (gy / N)).
 * Returns 1 if a label is out of range (the reference throws, src/mat/origin/cpu/nn/gather.cpp:58-87). */
int oracle_softmax_ce(const float *x, const int32_t *t, int64_t B, int64_t C, float *loss, float *dlogits)
{
    float *p = (float *)malloc(sizeof(float) * (size_t)B * (size_t)C);
    softmax_rows(x, p, B, C);
    float sum = 0.0f;
    for (int64_t i = 0; i < B; ++i)
    {
        if (t[i] < 0 || t[i] >= C)
        {
            free(p);
            return 1;
        }
        sum += logf(p[i * C + t[i]] + 1e-8f);
    }
    if (loss)
        *loss = -sum / (float)B;
    if (dlogits)
    {
        const float scale = 1.0f / (float)B;
        for (int64_t i = 0; i < B; ++i)
            for (int64_t c = 0; c < C; ++c)
            {
                float onehot       = (c == t[i]) ? 1.0f : 0.0f;
                dlogits[i * C + c] = (p[i * C + c] - onehot) * scale;
            }
    }
    free(p);
    return 0;
}

/* One Adam update of n elements at step count t (1-based), preceded by the WeightDecay hook when hook_wd > 0.
 * include/origin/optim/hooks.h:40-66: g += p * rate (in place, so g is an output too);
 * src/optim/adam.cpp:50-110, every intermediate rounded to fp32:
 *   m = m*b1 + g*(1-b1);  v = v*b2 + (g*g)*(1-b2);  mh = m * (1/(1-b1^t));  vh = v * (1/(1-b2^t));
 *   p = p - (mh / (powf(vh, 0.5) + eps)) * lr,  with b^t = std::pow(float b, float t) and (1-b1) computed in fp32. */
void oracle_adam_step(float *p, float *g, float *m, float *v, int64_t n, int t, float lr, float b1, float b2,
                      float eps, float hook_wd)
{
    const float one_m_b1 = 1.0f - b1, one_m_b2 = 1.0f - b2;
    const float b1p = powf(b1, (float)t), b2p = powf(b2, (float)t);
    const float mhs = 1.0f / (1.0f - b1p), vhs = 1.0f / (1.0f - b2p);
    for (int64_t i = 0; i < n; ++i)
    {
        if (hook_wd > 0.0f)
        {
            float term = p[i] * hook_wd;
            g[i]       = g[i] + term;
        }
        float gi = g[i];
        float a1 = m[i] * b1, a2 = gi * one_m_b1;
        m[i]     = a1 + a2;
        float gg = gi * gi;
        float c1 = v[i] * b2, c2 = gg * one_m_b2;
        v[i]     = c1 + c2;
        float mh = m[i] * mhs, vh = v[i] * vhs;
        float den = powf(vh, 0.5f) + eps;
        float upd = mh / den;
        float stp = upd * lr;
        p[i]      = p[i] - stp;
    }
}

/* One SGD update.  Hook first (hooks.h:40-66, in place on g), then src/optim/sgd.cpp:18-75:
 *   if wd > 0: g = g + p*wd;  if momentum > 0: buf = buf*momentum + g;  g = nesterov ? g + buf*momentum : buf;
 *   p = p - g*lr.  buf may be NULL when momentum == 0. */
void oracle_sgd_step(float *p, float *g, float *buf, int64_t n, float lr, float momentum, float wd, int nesterov,
                     float hook_wd)
{
    for (int64_t i = 0; i < n; ++i)
    {
        if (hook_wd > 0.0f)
        {
            float term = p[i] * hook_wd;
            g[i]       = g[i] + term;
        }
        float gi = g[i];
        if (wd > 0.0f)
        {
            float term = p[i] * wd;
            gi         = gi + term;
        }
        if (momentum > 0.0f)
        {
            float t1 = buf[i] * momentum;
            buf[i]   = t1 + gi;
            if (nesterov)
            {
                float t2 = buf[i] * momentum;
                gi       = gi + t2;
            }
            else
                gi = buf[i];
        }
        float stp = gi * lr;
        p[i]      = p[i] - stp;
    }
}

static int out_size(int in, int k, int s, int p)
{
    /* include/origin/utils/conv_utils.h:32-35 */
    return (in + 2 * p - k) / s + 1;
}

/* col[(n*OH+oh)*OW+ow, (c*KH+kh)*KW+kw] = x_padded[n, c, oh*S+kh, ow*S+kw]  (zero outside the image).
 * src/mat/origin/cpu/conv/conv2d.cpp:39-160 (im2col_impl, to_matrix = true). */
void oracle_im2col(const float *x, float *col, int64_t N, int64_t C, int64_t H, int64_t W, int KH, int KW, int S, int P)
{
    const int OH = out_size((int)H, KH, S, P), OW = out_size((int)W, KW, S, P);
    const int64_t cols = C * KH * KW;
    for (int64_t n = 0; n < N; ++n)
        for (int oh = 0; oh < OH; ++oh)
            for (int ow = 0; ow < OW; ++ow)
            {
                int64_t row = (n * OH + oh) * OW + ow;
                for (int64_t c = 0; c < C; ++c)
                    for (int kh = 0; kh < KH; ++kh)
                        for (int kw = 0; kw < KW; ++kw)
                        {
                            int h = oh * S + kh - P, w = ow * S + kw - P;
                            float v = 0.0f;
                            if (h >= 0 && h < H && w >= 0 && w < W)
                                v = x[((n * C + c) * H + h) * W + w];
                            col[row * cols + (c * KH + kh) * KW + kw] = v;
                        }
            }
}

/* Scatter-add of a column matrix back to the image; accumulation order kh, kw, oh, ow as the reference.
 * src/mat/origin/cpu/conv/conv2d.cpp:212-380 (col2im_impl, to_matrix = true). */
void oracle_col2im(const float *col, float *x, int64_t N, int64_t C, int64_t H, int64_t W, int KH, int KW, int S, int P)
{
    const int OH = out_size((int)H, KH, S, P), OW = out_size((int)W, KW, S, P);
    const int64_t cols = C * KH * KW;
    const int64_t PH = H + 2 * P, PW = W + 2 * P;
    float *pad = (float *)calloc((size_t)(N * C * PH * PW), sizeof(float));
    for (int64_t n = 0; n < N; ++n)
        for (int64_t c = 0; c < C; ++c)
            for (int kh = 0; kh < KH; ++kh)
                for (int kw = 0; kw < KW; ++kw)
                    for (int oh = 0; oh < OH; ++oh)
                        for (int ow = 0; ow < OW; ++ow)
                        {
                            int64_t row = (n * OH + oh) * OW + ow;
                            int h = oh * S + kh, w = ow * S + kw;
                            if (h < PH && w < PW)
                                pad[((n * C + c) * PH + h) * PW + w] += col[row * cols + (c * KH + kh) * KW + kw];
                        }
    for (int64_t n = 0; n < N; ++n)
        for (int64_t c = 0; c < C; ++c)
            for (int64_t h = 0; h < H; ++h)
                for (int64_t w = 0; w < W; ++w)
                    x[((n * C + c) * H + h) * W + w] = pad[((n * C + c) * PH + h + P) * PW + w + P];
    free(pad);
}

/* y[N,OC,OH,OW] = conv2d(x[N,C,H,W], w[OC,C,KH,KW]) + b via im2col . W^T, then NHWC -> NCHW.
 * src/mat/origin/cpu/conv/conv2d.cpp:404-515. */
void oracle_conv2d_forward(const float *x, const float *w, const float *b, float *y, int64_t N, int64_t C, int64_t H,
                           int64_t W, int64_t OC, int KH, int KW, int S, int P)
{
    const int OH = out_size((int)H, KH, S, P), OW = out_size((int)W, KW, S, P);
    const int64_t rows = N * OH * OW, cols = C * KH * KW;
    float *col = (float *)malloc(sizeof(float) * (size_t)(rows * cols));
    oracle_im2col(x, col, N, C, H, W, KH, KW, S, P);
    for (int64_t r = 0; r < rows; ++r)
    {
        int64_t n = r / ((int64_t)OH * OW), hw = r % ((int64_t)OH * OW);
        for (int64_t oc = 0; oc < OC; ++oc)
        {
            float sum = 0.0f;
            for (int64_t k = 0; k < cols; ++k)
                sum += col[r * cols + k] * w[oc * cols + k];
            if (b)
                sum = sum + b[oc];
            y[(n * OC + oc) * OH * OW + hw] = sum;
        }
    }
    free(col);
}

/* Gradients of conv2d for upstream gy[N,OC,OH,OW].  src/mat/origin/cpu/conv/conv2d.cpp:517-599.
 * mode 0 ("textbook"): gy is permuted NCHW -> [N*OH*OW, OC] before the two products, which is the gradient of the
 *         forward above (docs/design/operators_theory.md:1149-1155).
 * mode 1 ("reference layout"): gy's NCHW buffer is reinterpreted as [N*OH*OW, OC] without permuting, which is what
 *         the reference code does (conv2d.cpp:548 gy.reshape); identical to mode 0 when OC == 1 or OH*OW == 1.
 * gb = gy.sum(2).sum(2).sum(0) in both modes (:565-577), i.e. sums over oh, then ow, then n.
 * gx, gw, gb may each be NULL. */
void oracle_conv2d_backward(const float *gy, const float *x, const float *w, float *gx, float *gw, float *gb, int64_t N,
                            int64_t C, int64_t H, int64_t W, int64_t OC, int KH, int KW, int S, int P, int mode)
{
    const int OH = out_size((int)H, KH, S, P), OW = out_size((int)W, KW, S, P);
    const int64_t hw = (int64_t)OH * OW, rows = N * hw, cols = C * KH * KW;
    float *gyf = (float *)malloc(sizeof(float) * (size_t)(rows * OC));
    if (mode == 1)
        memcpy(gyf, gy, sizeof(float) * (size_t)(rows * OC));
    else
        for (int64_t n = 0; n < N; ++n)
            for (int64_t oc = 0; oc < OC; ++oc)
                for (int64_t i = 0; i < hw; ++i)
                    gyf[(n * hw + i) * OC + oc] = gy[(n * OC + oc) * hw + i];
    if (gw)
    {
        float *col = (float *)malloc(sizeof(float) * (size_t)(rows * cols));
        oracle_im2col(x, col, N, C, H, W, KH, KW, S, P);
        for (int64_t oc = 0; oc < OC; ++oc)
            for (int64_t k = 0; k < cols; ++k)
            {
                float sum = 0.0f;
                for (int64_t r = 0; r < rows; ++r)
                    sum += gyf[r * OC + oc] * col[r * cols + k];
                gw[oc * cols + k] = sum;
            }
        free(col);
    }
    if (gb)
    {
        /* sum over oh (axis 2), then ow (axis 2 of the result), then n (axis 0) */
        float *t1 = (float *)calloc((size_t)(N * OC * OW), sizeof(float));
        for (int64_t n = 0; n < N; ++n)
            for (int64_t oc = 0; oc < OC; ++oc)
                for (int ow = 0; ow < OW; ++ow)
                {
                    float s = 0.0f;
                    for (int oh = 0; oh < OH; ++oh)
                        s += gy[((n * OC + oc) * OH + oh) * OW + ow];
                    t1[(n * OC + oc) * OW + ow] = s;
                }
        for (int64_t oc = 0; oc < OC; ++oc)
        {
            float tot = 0.0f;
            for (int64_t n = 0; n < N; ++n)
            {
                float s = 0.0f;
                for (int ow = 0; ow < OW; ++ow)
                    s += t1[(n * OC + oc) * OW + ow];
                tot += s;
            }
            gb[oc] = tot;
        }
        free(t1);
    }
    if (gx)
    {
        float *gcol = (float *)malloc(sizeof(float) * (size_t)(rows * cols));
        for (int64_t r = 0; r < rows; ++r)
            for (int64_t k = 0; k < cols; ++k)
            {
                float sum = 0.0f;
                for (int64_t oc = 0; oc < OC; ++oc)
                    sum += gyf[r * OC + oc] * w[oc * cols + k];
                gcol[r * cols + k] = sum;
            }
        oracle_col2im(gcol, gx, N, C, H, W, KH, KW, S, P);
        free(gcol);
    }
    free(gyf);
}

/* ---- BatchNorm (2-D {N,C}: HW = 1; 4-D {N,C,H,W}: HW = H*W) and SiLU -----------------------------------------------
 * Follows cpu::batch_norm_forward (src/mat/origin/cpu/normalization/batch_norm.cpp:20-236): training statistics are
 * two sequential passes per channel (mean, then the mean of squared differences -- the BIASED variance); in
 * evaluation mode mean/var are copies of the running statistics; x_norm = (x - mean) / sqrt(var + eps);
 * y = gamma * x_norm + beta. */
void oracle_batch_norm_forward(const float *x, const float *gamma, const float *beta, const float *running_mean,
                               const float *running_var, int training, float eps, int64_t N, int64_t C, int64_t HW,
                               float *y, float *mean, float *var, float *x_norm)
{
    for (int64_t c = 0; c < C; ++c)
    {
        if (training)
        {
            float sum = 0.0f;
            for (int64_t n = 0; n < N; ++n)
                for (int64_t i = 0; i < HW; ++i)
                    sum += x[(n * C + c) * HW + i];
            const float count = (float)(N * HW);
            mean[c]           = sum / count;
            float sq          = 0.0f;
            for (int64_t n = 0; n < N; ++n)
                for (int64_t i = 0; i < HW; ++i)
                {
                    const float d = x[(n * C + c) * HW + i] - mean[c];
                    sq += d * d;
                }
            var[c] = sq / count;
        }
        else
        {
            mean[c] = running_mean[c];
            var[c]  = running_var[c];
        }
    }
    for (int64_t n = 0; n < N; ++n)
        for (int64_t c = 0; c < C; ++c)
        {
            const float sd = sqrtf(var[c] + eps);
            for (int64_t i = 0; i < HW; ++i)
            {
                const int64_t idx = (n * C + c) * HW + i;
                const float xn    = (x[idx] - mean[c]) / sd;
                if (x_norm)
                    x_norm[idx] = xn;
                y[idx] = gamma[c] * xn + beta[c];
            }
        }
}

/* cpu::batch_norm_backward (batch_norm.cpp:252-415): dbeta = sum gy, dgamma = sum gy * x_norm,
 * gx = (gamma / std) * (gy - mean(gy) - x_norm * mean(gy * x_norm)), whatever the mode of the forward pass. */
void oracle_batch_norm_backward(const float *gy, const float *gamma, const float *saved_var, const float *x_norm,
                                float eps, int64_t N, int64_t C, int64_t HW, float *gx, float *dgamma, float *dbeta)
{
    for (int64_t c = 0; c < C; ++c)
    {
        float sum_gy = 0.0f, sum_gx = 0.0f;
        for (int64_t n = 0; n < N; ++n)
            for (int64_t i = 0; i < HW; ++i)
            {
                const int64_t idx = (n * C + c) * HW + i;
                sum_gy += gy[idx];
                sum_gx += gy[idx] * x_norm[idx];
            }
        const float count = (float)(N * HW);
        const float mg = sum_gy / count, mgx = sum_gx / count;
        const float sd = sqrtf(saved_var[c] + eps);
        dgamma[c]      = sum_gx;
        dbeta[c]       = sum_gy;
        for (int64_t n = 0; n < N; ++n)
            for (int64_t i = 0; i < HW; ++i)
            {
                const int64_t idx = (n * C + c) * HW + i;
                gx[idx]           = (gamma[c] / sd) * (gy[idx] - mg - x_norm[idx] * mgx);
            }
    }
}

/* nn::BatchNorm2d::forward's update after a training step (src/nn/layers/batch_norm2d.cpp:66-83):
 * running = momentum * running + (1 - momentum) * current  -- momentum weighs the OLD value, default 0.1. */
void oracle_batch_norm_update_running(float *running_mean, float *running_var, const float *mean, const float *var,
                                      float momentum, int64_t C)
{
    for (int64_t c = 0; c < C; ++c)
    {
        running_mean[c] = momentum * running_mean[c] + (1.0f - momentum) * mean[c];
        running_var[c]  = momentum * running_var[c] + (1.0f - momentum) * var[c];
    }
}

/* cpu::silu / cpu::silu_backward (src/mat/origin/cpu/activation/silu.cpp:48-92). */
void oracle_silu_forward(const float *x, float *y, int64_t n)
{
    for (int64_t i = 0; i < n; ++i)
    {
        const float s = 1.0f / (1.0f + expf(-x[i]));
        y[i]          = x[i] * s;
    }
}

void oracle_silu_backward(const float *gy, const float *x, float *gx, int64_t n)
{
    for (int64_t i = 0; i < n; ++i)
    {
        const float v = x[i];
        const float s = 1.0f / (1.0f + expf(-v));
        gx[i]         = gy[i] * (s + v * s * (1.0f - s));
    }
}
