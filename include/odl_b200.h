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

/* GEMM arithmetic: 3xTF32 (default, fp32-class accuracy: three tf32 MMAs per product) or plain TF32. */
#define ODL_PRECISION_3XTF32 0
#define ODL_PRECISION_TF32 1

/* epilogue flags of odl_gemm_ex, applied in this order to each result value v at (m, n) */
#define ODL_EPI_BIAS 1    /* v += bias[n]                                   */
#define ODL_EPI_RELU 2    /* v  = v > 0 ? v : 0                             */
#define ODL_EPI_MASK 4    /* v  = mask_src[m,n] > 0 ? v : 0  (ReLU backward) */
#define ODL_EPI_COLSUM 8  /* colsum[n] += v  (caller zeroes colsum)          */
#define ODL_EPI_SMALL 16  /* also write D_small = tf32(v - trunc_tf32(v))    */

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

#ifdef __cplusplus
}
#endif
#endif /* ODL_B200_H_ */
