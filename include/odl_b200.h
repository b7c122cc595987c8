/*
 * odl_b200 -- C ABI of the B200 (sm_100a) dense hot path for OriginDL.
 *
 * Every entry point takes plain device pointers (fp32 unless stated), int64 sizes, int flags and a CUDA stream
 * passed as void* (cudaStream_t; NULL = default stream), and returns an int status (ODL_OK = 0).  On a non-zero
 * status odl_last_error() holds a message; a C++ host maps it to the exception the reference would throw
 * (THROW_RUNTIME_ERROR / THROW_INVALID_ARG, include/origin/utils/exception.h:37-60).
 * Matrices are row-major and contiguous in their last dimension, like OriginMat storage.
 *
 * Each declaration names the reference interface it stands in for (paths relative to the OriginDL tree).
 * There is no CPU fallback behind any of these: without a CUDA device they fail with ODL_ERR_CUDA.
 */
#ifndef ODL_B200_H_
#define ODL_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* status codes */
#define ODL_OK 0
#define ODL_ERR_INVALID_ARGUMENT 1
#define ODL_ERR_MISALIGNED 2
#define ODL_ERR_CUDA 3
#define ODL_ERR_KERNEL_TIMEOUT 4
#define ODL_ERR_TOO_LARGE 5
#define ODL_ERR_NOT_INITIALIZED 6
#define ODL_ERR_STALE_GRAPH 7 /* a recorded step graph refers to scratch memory that was replaced since: capture again */
#define ODL_ERR_COMM 8          /* the communicator reported an error, NCCL is unavailable, or it was aborted earlier */
#define ODL_ERR_COMM_TIMEOUT 9  /* a collective did not complete within the watchdog's limit; communicator aborted */

/* GEMM arithmetic: 3xTF32 (default, fp32-class accuracy: three tf32 MMAs per product) or plain TF32. */
#define ODL_PRECISION_3XTF32 0
#define ODL_PRECISION_TF32 1

/* epilogue flags of odl_gemm_ex, applied in this order to each result value v at (m, n) */
#define ODL_EPI_BIAS 1    /* v += bias[n]                                   */
#define ODL_EPI_RELU 2    /* v  = v > 0 ? v : 0                             */
#define ODL_EPI_MASK 4    /* v  = mask_src[m,n] > 0 ? v : 0  (ReLU backward) */
#define ODL_EPI_COLSUM 8  /* colsum[n] += v  (caller zeroes colsum)          */
#define ODL_EPI_SMALL 16  /* also write D_small = tf32(v - trunc_tf32(v))    */

/* activations fused after conv2d / BatchNorm */
#define ODL_ACT_NONE 0
#define ODL_ACT_RELU 1
#define ODL_ACT_SILU 2

/* weight layouts of the Linear entry points */
#define ODL_W_OUT_IN 0 /* W is [out, in]: functional::custom_linear / LinearOp (include/origin/operators/custom/linear.h:13-15) */
#define ODL_W_IN_OUT 1 /* W is {in, out}: nn::Linear (src/nn/layers/linear.cpp:39-48)                                       */

/* ---- library state ------------------------------------------------------------------------------------------ */

/* Bind the calling thread to `device`, resolve the tensor-map encoder and allocate the per-device error flag and
 * scratch arena.  Must be called once per process/device before anything else.
 * Stands in for the lazy CUDA set-up the reference does in origin::cuda (src/mat/origin/cuda/cuda_utils.cu). */
int odl_init(int device);

/* Message of the last non-zero status returned on this thread. */
const char *odl_last_error(void);

/* Synchronise `stream` and report whether any kernel gave up on a bounded wait since the last call
 * (ODL_ERR_KERNEL_TIMEOUT); the flag is cleared.  The counterpart of CUDA_CHECK_ASYNC
 * (include/origin/mat/origin/cuda/cuda_utils.cuh:14-33). */
int odl_device_status(void *stream);

/* Bytes currently held by the library's device scratch arena (operand splits, padded copies, im2col columns). */
int64_t odl_scratch_bytes(void);

/* Counts how often the library has replaced one of its scratch blocks (the arena above or the column-sum scratch) by a
 * larger one.  Anything that recorded kernel launches of this library into a CUDA graph holds raw addresses inside
 * those blocks; when this number differs from its value at recording time the graph must be recorded again
 * (odl_mlp_replay checks this itself and returns ODL_ERR_STALE_GRAPH).  No counterpart in the reference. */
long long odl_scratch_generation(void);

/* Number of kernels this library has launched in the process so far (a benchmark reports the delta over its timed
 * region).  No counterpart in the reference. */
long long odl_launch_count(void);

/* ---- GEMM ---------------------------------------------------------------------------------------------------- */

/* C[M,N] = A[M,K] . B[K,N].  Replaces origin::cuda::matmul (include/origin/mat/origin/cuda/cuda_ops.cuh:264,
 * src/mat/origin/cuda/math/mat_mul.cu:1833-1970) for 2-D fp32 operands; `batch` > 1 gives the 3-D x 2-D
 * (b_batched = 0) and 3-D x 3-D (b_batched = 1) forms the reference loops over on the host (mat_mul.cu:1920-1949). */
int odl_matmul(const float *A, const float *B, float *C, int64_t M, int64_t N, int64_t K, int64_t batch,
               int b_batched, int precision, void *stream);

/* D[M,N] = op(A)[M,K] . op(B)[K,N] with fused epilogue.  transA: A is stored [K,M]; transB: B is stored [N,K].
 * The combinations cover MatMul::backward (src/operators/math/mat_mul.cpp:123-182: gx = gy.W^T, gw = x^T.gy)
 * without the two materialised transposes the reference makes (src/mat/origin/cuda/shape/transpose.cu:191-221).
 * A_small / B_small: optional precomputed low parts for ODL_PRECISION_3XTF32 (same layout and pitch as A / B);
 * NULL lets the library compute them into scratch.  D_small, bias, mask_src, colsum are used per epilogue flag. */
int odl_gemm_ex(int transA, int transB, int64_t M, int64_t N, int64_t K, const float *A, const float *A_small,
                int64_t lda, const float *B, const float *B_small, int64_t ldb, float *D, float *D_small, int64_t ldd,
                const float *bias, const float *mask_src, int64_t ld_mask, float *colsum, int epilogue_flags,
                int precision, void *stream);

/* dst_small[r,c] = tf32(v - trunc_tf32(v)) with v = src[r,c] (masked by mask_src > 0 when given); optional padded
 * copy dst_big and column sums.  The operand-preparation pass of the 3xTF32 GEMM, exposed for callers that keep
 * low parts resident (weights after an optimizer step). No counterpart in the reference (it has no tensor-core path). */
int odl_split_tf32(const float *src, int64_t ld_src, int64_t rows, int64_t cols, const float *mask_src, int64_t ld_mask,
                   float *dst_big, float *dst_small, int64_t ld_dst, float *colsum, void *stream);

/* ---- Linear ------------------------------------------------------------------------------------------------- */

/* y[M,N] = relu?(x[M,K] . op(W) + b) in one kernel (GEMM with bias / ReLU epilogue).
 * w_layout ODL_W_OUT_IN replaces LinearOp::forward / functional::custom_linear (src/operators/custom/linear.cpp:12-144);
 * ODL_W_IN_OUT replaces nn::Linear::forward = mat_mul + broadcast_to + add (src/nn/layers/linear.cpp:80-106), and with
 * relu != 0 also the following functional::relu (src/operators/activation/relu.cpp:13-35; MLP::forward,
 * src/nn/models/mlp.cpp:43-61).  b may be NULL.  x_small / w_small: optional resident low parts (3xTF32);
 * y_small: optional output, the low part of y for the next layer's GEMM. */
int odl_linear_forward(const float *x, const float *x_small, const float *w, const float *w_small, const float *b,
                       float *y, float *y_small, int64_t M, int64_t N, int64_t K, int w_layout, int relu, int precision,
                       void *stream);

/* Gradients of the layer above for upstream dy[M,N]:  g = y ? dy * (y > 0) : dy;  db[N] = colsum(g);
 * dx[M,K] = g . W;  dW = g^T . x (same layout as W).  The rule LinearOp::backward leaves unimplemented
 * (src/operators/custom/linear.cpp:116-121), equal to the chain ReLU::backward (relu.cpp:37-54) ->
 * Add::backward / BroadcastTo::backward -> sum_to (src/operators/math/add.cpp:29-55, broadcast_to.cpp:29-46) ->
 * MatMul::backward (src/operators/math/mat_mul.cpp:123-182).  y is the forward OUTPUT when the layer had a ReLU, else NULL.
 * dx, dw, db may each be NULL (not computed). */
int odl_linear_backward(const float *x, const float *x_small, const float *w, const float *w_small, const float *dy,
                        const float *y, float *dx, float *dw, float *db, int64_t M, int64_t N, int64_t K, int w_layout,
                        int precision, void *stream);

/* Same, for a layer inside an MLP: the dx GEMM's epilogue already applies the PREVIOUS layer's ReLU mask
 * (prev_y[M,K] > 0), sums the previous layer's bias gradient prev_db[K] and emits dx_small, so the previous layer's
 * backward needs no preparation pass of its own (pass its y = NULL and db = NULL there, dx here as its dy and
 * dx_small here as its dy_small).  dy_small is the 3xTF32 low part of dy when the caller already holds it (the
 * dx_small of the layer above); NULL makes this call compute it.
 * No counterpart in the reference (it runs these as separate kernels). */
int odl_linear_backward_chain(const float *x, const float *x_small, const float *w, const float *w_small, const float *dy, const float *dy_small,
                              const float *y, float *dx, float *dx_small, const float *prev_y, float *prev_db, float *dw,
                              float *db, int64_t M, int64_t N, int64_t K, int w_layout, int precision, void *stream);

/* ---- element-wise pieces of the operator API -------------------------------------------------------------------- */

/* y = x > 0 ? x : 0.  Replaces origin::cuda::relu (include/origin/mat/origin/cuda/cuda_ops.cuh:186). */
int odl_relu_forward(const float *x, float *y, int64_t n, void *stream);
/* gx = gy * (x_or_y > 0).  Replaces gt + multiply of ReLU::backward (cuda_ops.cuh:125,:75; relu.cpp:37-54). */
int odl_relu_backward(const float *gy, const float *x_or_y, float *gx, int64_t n, void *stream);
/* y[m,n] = x[m,n] + b[n].  Replaces broadcast_to + add (cuda_ops.cuh:304,:57) as used by nn::Linear. */
int odl_add_bias(const float *x, const float *b, float *y, int64_t M, int64_t N, void *stream);
/* out[n] = sum_m g[m,n].  Replaces origin::cuda::sum_to for {M,N} -> {1,N} (cuda_ops.cuh:312;
 * src/mat/origin/cuda/math/sum_to.cu:19-91), without its N <= 1024 launch limit (sum.cu:284-287). */
int odl_sum_to_row(const float *g, float *out, int64_t M, int64_t N, void *stream);

/* out = x (op) y for same-shape tensors: op 0 add, 1 subtract, 2 multiply.  Replaces origin::cuda::add / subtract /
 * multiply (cuda_ops.cuh:57,:66,:75) as used by Add, Sub, Mul operators and by gradient accumulation. */
int odl_binary(int op, const float *x, const float *y, float *out, int64_t n, void *stream);
/* out = x * alpha (tensor times 0-dim scalar, src/operators/math/mul.cpp:113-117). */
int odl_scale(const float *x, float alpha, float *out, int64_t n, void *stream);
/* y += alpha * x with the product rounded first: add_inplace of a scaled tensor, i.e. the WeightDecay hook
 * (include/origin/optim/hooks.h:52-64) and TensorImpl's gradient accumulation (src/core/tensor_impl.cpp:186-196). */
int odl_axpy(float alpha, const float *x, float *y, int64_t n, void *stream);
/* out[i] = value.  Replaces the factory kernels behind Tensor::zeros / ones / full (src/mat/origin/cuda/factory.cu). */
int odl_fill(float *out, float value, int64_t n, void *stream);
/* out[0] = sum of all elements, fixed order.  Replaces origin::cuda::sum with axis = -1 (cuda_ops.cuh:273). */
int odl_sum_all(const float *x, float *out, int64_t n, void *stream);

/* ---- loss ------------------------------------------------------------------------------------------------------- */

/* loss[0] = -(1/B) sum_i log(softmax(logits)[i,t_i] + 1e-8) and/or dlogits = (softmax - onehot) * grad_scale / B, both
 * on the device in two launches and without host synchronisation.  Replaces SoftmaxCrossEntropy::forward/backward
 * (src/operators/loss/softmax_cross_entropy.cpp:17-111, ~25 kernels and two .item() syncs).  labels: int32 or int64
 * (labels_are_int64); an out-of-range label is reported by odl_device_status as ODL_ERR_INVALID_ARGUMENT (the
 * reference throws from gather, src/mat/origin/cpu/nn/gather.cpp:58-87).  loss or dlogits may be NULL. */
int odl_softmax_cross_entropy(const float *logits, const void *labels, int labels_are_int64, int64_t B, int64_t C,
                              float *loss, float *dlogits, float grad_scale, void *stream);

/* Same computation as odl_softmax_cross_entropy for callers that cannot allocate device memory once they are running
 * (a host application that gave the whole GPU to its own pool at start-up; a latency-critical loop that cannot take
 * the device-wide synchronisation of an allocation).  It has no counterpart in the reference.  The per-row scratch the
 * loss needs lives in a fixed 256 KiB array inside the library image (held by every GPU that loads the library until
 * the process exits) instead of the growable arena, so the call itself performs no allocation of any kind.
 * Limits: B <= ODL_STATIC_SOFTMAX_MAX_ROWS, else ODL_ERR_TOO_LARGE.  The first call on a device resolves the array's
 * device address with the device current at that moment (cudaGetSymbolAddress).  CUDA loads a library's device code
 * lazily, so that look-up is also what places the array's 256 KiB on the GPU: make the first call (any small batch)
 * during start-up, before the host's own pool takes the remaining memory and before any stream capture; every later call
 * on that device touches no allocator at all.  All calls share
 * the one array, which keeps the previous call's contents: nothing in it needs clearing (every call overwrites the
 * rows it reads), but two calls that overlap on the GPU race on it -- keep them on one stream. */
#define ODL_STATIC_SOFTMAX_MAX_ROWS 65536
int odl_softmax_cross_entropy_static(const float *logits, const void *labels, int labels_are_int64, int64_t B, int64_t C,
                                     float *loss, float *dlogits, float grad_scale, void *stream);

/* ---- optimizers -------------------------------------------------------------------------------------------------- */

/* One fused in-place Adam update of n contiguous parameters at step t (1-based), same operation order and fp32 rounding
 * as Adam::step_one (src/optim/adam.cpp:19-114) preceded by the WeightDecay hook (include/origin/optim/hooks.h:40-66;
 * grad += hook_weight_decay * param, written back to grad) when hook_weight_decay > 0.  grad_scale multiplies the
 * gradient first (1/world_size after a summing all-reduce; 1 otherwise).  param_small: optional output, low part of
 * the updated parameters for the next 3xTF32 GEMM. */
int odl_adam_step(float *param, float *grad, float *m, float *v, float *param_small, int64_t n, int t, float lr,
                  float beta1, float beta2, float eps, float hook_weight_decay, float grad_scale, void *stream);

/* One fused in-place SGD update: SGD::step_one (src/optim/sgd.cpp:18-75) with weight_decay, momentum and Nesterov,
 * after the optional WeightDecay hook.  momentum_buf may be NULL when momentum == 0. */
int odl_sgd_step(float *param, float *grad, float *momentum_buf, float *param_small, int64_t n, float lr, float momentum,
                 float weight_decay, int nesterov, float hook_weight_decay, float grad_scale, void *stream);

/* ---- Conv2d (im2col + GEMM) -------------------------------------------------------------------------------------- */

/* col[N*OH*OW, C*KH*KW] from x[N,C,H,W]; replaces origin::cuda::im2col (cuda_ops.cuh:335; conv2d.cu:32,:255,:417)
 * without the padded image copy.  C*KH*KW must be a multiple of 4 in this public row-matrix form. */
int odl_im2col(const float *x, float *col, int64_t N, int64_t C, int64_t H, int64_t W, int KH, int KW, int stride, int pad,
               void *stream);
/* x[N,C,H,W] = scatter-add of col; replaces origin::cuda::col2im (cuda_ops.cuh:349; conv2d.cu:146,:322) with a gather
 * that needs no atomics. */
int odl_col2im(const float *col, float *x, int64_t N, int64_t C, int64_t H, int64_t W, int KH, int KW, int stride, int pad,
               void *stream);
/* y[N,OC,OH,OW] = act(conv2d(x, w[OC,C,KH,KW]) + b), act = ODL_ACT_NONE / ODL_ACT_RELU / ODL_ACT_SILU.  Replaces
 * origin::cuda::conv2d (cuda_ops.cuh:363; src/mat/origin/cuda/conv/conv2d.cu:563-678): im2col, one GEMM whose epilogue
 * adds the bias, applies the activation and writes NCHW directly. */
int odl_conv2d_forward(const float *x, const float *w, const float *b, float *y, int64_t N, int64_t C, int64_t H,
                       int64_t W, int64_t OC, int KH, int KW, int stride, int pad, int act, int precision, void *stream);
/* The inference block conv -> BatchNorm2d (evaluation mode) -> ReLU / SiLU of the reference's CNN examples
 * (tests/example/mnist/conv_mnist.cpp; the YOLOv5 Conv block) as ONE GEMM: y = act(scale[oc] * conv2d(x, w) + shift[oc])
 * with scale / shift from odl_batch_norm_fold.  Replaces origin::cuda::conv2d + origin::cuda::batch_norm
 * (src/mat/origin/cuda/normalization/batch_norm.cu) + relu / silu, i.e. three passes over the activation. */
int odl_conv2d_bn_act_forward(const float *x, const float *w, const float *scale, const float *shift, float *y, int64_t N,
                              int64_t C, int64_t H, int64_t W, int64_t OC, int KH, int KW, int stride, int pad, int act,
                              int precision, void *stream);
/* gx, gw, gb for upstream gy[N,OC,OH,OW]; replaces origin::cuda::conv2d_backward (cuda_ops.cuh:376; conv2d.cu:680-765).
 * gy_layout 0: gy is permuted to [N*OH*OW, OC] (the gradient of the forward pass); 1: the NCHW buffer is
 * reinterpreted as [N*OH*OW, OC] exactly as the reference does (conv2d.cu:714).  gx, gw, gb may each be NULL. */
int odl_conv2d_backward(const float *gy, const float *x, const float *w, float *gx, float *gw, float *gb, int64_t N,
                        int64_t C, int64_t H, int64_t W, int64_t OC, int KH, int KW, int stride, int pad, int gy_layout,
                        int precision, void *stream);

/* ---- BatchNorm (+ activation), SiLU ---------------------------------------------------------------------------------- */

/* y = act(gamma[c] * (x - mean[c]) / sqrt(var[c] + eps) + beta[c]) over x[N, C, HW] (HW = H*W; HW = 1 is the {N, C}
 * form of BatchNorm1d).  Replaces cpu/cuda::batch_norm_forward (src/mat/origin/cpu/normalization/batch_norm.cpp:20-236,
 * src/mat/origin/cuda/normalization/batch_norm.cu) and the activation that follows it.
 * training != 0: mean / var are the batch mean and BIASED variance, written to save_mean / save_var[C] (required);
 *   when running_mean / running_var are given they are updated in place the way nn::BatchNorm2d does after the
 *   operator (src/nn/layers/batch_norm2d.cpp:66-83): running = momentum * running + (1 - momentum) * batch.
 * training == 0: mean / var are running_mean / running_var (required; copied to save_* when those are given).
 * The reference also materialises x_norm for backward; this library does not (backward recomputes it). */
int odl_batch_norm_forward(const float *x, const float *gamma, const float *beta, float *running_mean,
                           float *running_var, int training, float eps, float momentum, int64_t N, int64_t C, int64_t HW,
                           int act, float *y, float *save_mean, float *save_var, void *stream);
/* With g = gy * act'(z), z the pre-activation: dbeta = sum g, dgamma = sum g * x_norm,
 * gx = gamma / std * (g - mean(g) - x_norm * mean(g * x_norm)) -- cpu::batch_norm_backward (batch_norm.cpp:252-415),
 * which the reference applies whatever the mode of the forward pass; after a training-mode forward it is the exact
 * gradient (there the reference's own operator throws, src/operators/normalization/batch_norm.cpp:78-92). */
int odl_batch_norm_backward(const float *gy, const float *x, const float *gamma, const float *beta, const float *save_mean,
                            const float *save_var, float eps, int64_t N, int64_t C, int64_t HW, int act, float *gx,
                            float *dgamma, float *dbeta, void *stream);
/* scale = gamma / sqrt(var + eps), shift = beta + scale * (bias - mean) (bias may be NULL): evaluation-mode BatchNorm
 * as a per-channel affine map for odl_conv2d_bn_act_forward.  No counterpart in the reference. */
int odl_batch_norm_fold(const float *gamma, const float *beta, const float *mean, const float *var, const float *bias,
                        float eps, int64_t C, float *scale, float *shift, void *stream);
/* y = x / (1 + exp(-x)); gx = gy * (s + x * s * (1 - s)), s = 1 / (1 + exp(-x)).  Replaces cpu/cuda::silu and
 * silu_backward (src/mat/origin/cpu/activation/silu.cpp:48-92). */
int odl_silu_forward(const float *x, float *y, int64_t n, void *stream);
int odl_silu_backward(const float *gy, const float *x, float *gx, int64_t n, void *stream);

/* ---- MLP training state (nn::MLP + loss + autograd + optimizer, device-resident) ----------------------------- */

/* Build an MLP with layer widths sizes[0..n_sizes) (ReLU after every layer but the last, like nn::MLP,
 * src/nn/models/mlp.cpp:11-61) for a fixed batch, with its optimizer: 0 = SGD(lr, momentum), 1 = Adam(lr, 0.9, 0.999,
 * 1e-8); hook_weight_decay > 0 adds the WeightDecay hook (tests/example/mnist/mlp_mnist.cpp:406-408).  Parameters,
 * gradients and optimizer state live in flat device buffers allocated here, once. */
int odl_mlp_create(const int32_t *sizes, int n_sizes, int64_t batch, int optimizer, float lr, float momentum,
                   float hook_weight_decay, int precision, void **handle);
int odl_mlp_destroy(void *handle);
/* Number of parameters in packed form (sum of in*out + out). */
int64_t odl_mlp_param_count(void *handle);
/* Install parameters from a packed HOST array [W_0 {in,out}, b_0 {1,out}, W_1, ...] (the order of
 * Module::named_parameters: layer_i.weight, layer_i.bias); resets the optimizer state. */
int odl_mlp_set_params(void *handle, const float *host_packed, void *stream);
/* Copy parameters (which = 0), the gradients of the last backward (1), the first-moment / momentum buffer (2) or
 * Adam's second moment (3) to a packed HOST array. */
int odl_mlp_get_packed(void *handle, int which, float *host_packed, void *stream);
/* Restore optimizer state read with odl_mlp_get_packed(2 / 3) and odl_mlp_step_count (call after odl_mlp_set_params,
 * which zeroes it).  The reference's checkpoint omits optimizer state (src/io/checkpoint.cpp:38-43: the optimizer.odl
 * path is computed and never written); with it a resumed run continues the SAME trajectory. */
int odl_mlp_set_optimizer_state(void *handle, const float *m_packed, const float *v_packed, int step_count, void *stream);
/* Optimizer steps taken since odl_mlp_set_params (Adam's t, src/optim/adam.cpp:49-50). */
int64_t odl_mlp_step_count(void *handle);
/* model(x) and softmax_cross_entropy(y, t) for x[batch, sizes[0]] and labels[batch] on the device; also starts the
 * backward pass (d loss / d logits and the head's bias gradient). */
int odl_mlp_forward_loss(void *handle, const float *x, const void *labels, int labels_are_int64, void *stream);
/* loss.backward(), one layer at a time from the head (layer = L-1) down to 0, so that a data-parallel caller can
 * all-reduce layer l's gradient bucket while layer l-1 is still computing. */
int odl_mlp_backward_layer(void *handle, int layer, void *stream);
/* optimizer.step(): one fused launch over the flat buffers; grad_scale multiplies the gradients first. */
int odl_mlp_optimizer_step(void *handle, float grad_scale, void *stream);
/* The same update for the parameters of one layer only (call once per layer and step, any order; first_of_step != 0
 * on the first call of a step advances the step counter all layers share).  A data-parallel caller updates each layer
 * as soon as its gradient bucket is reduced, so that the early layers' updates overlap the last bucket's all-reduce. */
int odl_mlp_optimizer_step_layer(void *handle, int layer, float grad_scale, int first_of_step, void *stream);
/* forward_loss + backward of every layer + optimizer_step. */
int odl_mlp_train_step(void *handle, const float *x, const void *labels, int labels_are_int64, void *stream);
/* Whole-step CUDA graph (the host overhead of Operator::operator() / TensorImpl::backward, src/core/tensor_impl.cpp:101-203,
 * is the dominant cost at small batch sizes): odl_mlp_capture records forward + loss + backward on the given STATIC device
 * buffers x[batch, sizes[0]] / labels[batch] into one graph (stream must be a non-default stream; one un-recorded pass
 * runs first to size scratch memory, parameters and optimizer state stay untouched); odl_mlp_replay runs one optimisation
 * step from it (graph launch + optimizer launch).  The caller refills x / labels in place between replays.
 * The graph holds addresses inside the library's scratch blocks.  Any later call that makes those blocks grow (a forward
 * at a larger batch, a conv layer, a second model) replaces them; odl_mlp_replay then launches nothing and returns
 * ODL_ERR_STALE_GRAPH until odl_mlp_capture has recorded the step again. */
int odl_mlp_capture(void *handle, const float *x, const void *labels, int labels_are_int64, void *stream);
int odl_mlp_replay(void *handle, void *stream);
/* Device pointers to the scalar loss and to the logits [batch, sizes[n-1]] of the last forward. */
float *odl_mlp_loss_ptr(void *handle);
float *odl_mlp_logits_ptr(void *handle);
/* Contiguous device range [dW_layer, db_layer] of the flat gradient buffer (layer = -1: the whole buffer). */
int odl_mlp_grad_bucket(void *handle, int layer, float **ptr, int64_t *count);

/* ---- data-parallel training: communicator, overlapped gradient all-reduce, failure detection ------------------------- */

/* The reference has no multi-GPU path (no collective, stream or peer copy anywhere in its tree); these entry points are
 * the new layer the data-parallel MLP step needs.  One process (or host thread) per GPU; every rank holds full replicas
 * of the parameters and optimizer state and its own rows of the batch; after the backward of layer l the contiguous
 * gradient range [dW_l, db_l] is summed over all ranks with ncclAllReduce on a stream of its own while layers l-1 ... 0
 * are still computing, and the fused optimizer scales by 1 / world.  NCCL is bound at run time (dlopen of "libnccl.so.2",
 * or of the path in the environment variable ODL_NCCL_LIBRARY): the library itself links only the CUDA runtime. */

#define ODL_COMM_UNIQUE_ID_BYTES 128
/* Rank 0 makes the 128-byte rendezvous token (ncclGetUniqueId) and hands it to the other ranks by any host channel. */
int odl_comm_unique_id(void *id_bytes);
/* Join the communicator described by the token (ncclCommInitRank; collective over all `world` ranks; the calling thread's
 * current CUDA device is the rank's GPU). */
int odl_comm_create(const void *id_bytes, int rank, int world, void **comm);
int odl_comm_destroy(void *comm);
/* buf[0..count) = sum over ranks, in place, enqueued on `stream`. */
int odl_comm_allreduce(void *comm, float *buf, int64_t count, void *stream);
/* Errors NCCL noticed asynchronously (ncclCommGetAsyncError): ODL_OK or ODL_ERR_COMM.  The counterpart, for
 * collectives, of CUDA_CHECK_ASYNC (include/origin/mat/origin/cuda/cuda_utils.cuh:14-33). */
int odl_comm_status(void *comm);
/* Host watchdog: polls done(arg) (non-zero = the watched work has completed) and odl_comm_status until completion, an
 * error, or timeout_ms.  On error / time-out the communicator is aborted (kernels waiting for a peer that never joined
 * end, the CUDA context stays usable) and ODL_ERR_COMM / ODL_ERR_COMM_TIMEOUT is returned; every later call on that
 * communicator returns ODL_ERR_COMM. */
int odl_comm_watch(void *comm, int timeout_ms, int (*done)(void *), void *arg);

/* Attach a communicator to an MLP (the handle does not take ownership).  dw0_panels (1..8) splits the weight gradient of
 * layer 0 -- the last GEMM of backward, whose all-reduce would otherwise overlap nothing -- into that many row panels,
 * each reduced while the next one is computed; 0 lets the library choose. */
int odl_mlp_dp_attach(void *handle, void *comm, int dw0_panels);
/* One data-parallel optimisation step on this rank's rows x[batch, sizes[0]]: forward, loss, backward with the overlapped
 * per-layer all-reduce (each layer's weight gradient is computed before its input gradient, so that its bucket's all-reduce
 * starts behind the dW GEMM), and on the library's communication stream each layer's fused update as soon as its bucket is
 * reduced and its input-gradient GEMM has finished; `stream` waits for that stream at the end.  Everything is enqueued;
 * the call does not wait for the GPU.  Environment variable ODL_DP_TRACE=1 prints the step's timeline (timing events on
 * both streams) to stderr and synchronises after every step. */
int odl_mlp_train_step_dp(void *handle, const float *x, const void *labels, int labels_are_int64, void *stream);
/* Watchdog over the last enqueued data-parallel step (odl_comm_watch on the end of its communication stream: the last
 * all-reduce and update). */
int odl_mlp_dp_wait(void *handle, int timeout_ms);

/* ---- input pipeline --------------------------------------------------------------------------------------------- */

/* Batch assembly from a data set resident in device memory: dst[i, 0:cols] = src[idx[i], 0:cols] and (when
 * labels_dst != NULL) labels_dst[i] = labels_src[idx[i]], i < n_idx; idx, labels are int64 DEVICE arrays, 0 <= idx[i]
 * < n_src (a violation writes zeros / -1 and is reported by odl_device_status).  Replaces the per-sample host loop of
 * DataLoader::next (src/data/dataloader.cpp:38-139) followed by the host-to-device copy of the batch. */
int odl_gather_rows(const float *src, int64_t ld_src, int64_t n_src, const int64_t *idx, int64_t n_idx, int64_t cols,
                    float *dst, int64_t ld_dst, const int64_t *labels_src, int64_t *labels_dst, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* ODL_B200_H_ */
