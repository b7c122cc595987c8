// Cross-translation-unit declarations of the library (host side).
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "gemm_tc.cuh"

namespace odl
{

bool is_ready();

// Scratch arena (one device block, bump-allocated, reset at the start of every top-level call).
void arena_reset();
int arena_reserve(size_t total_bytes);
void *arena_alloc(size_t bytes);
// Counts replacements of library-owned scratch blocks (arena, column-sum scratch): recorded graphs compare it.
long long scratch_generation();
void bump_scratch_generation();

size_t operand_scratch(const float *ptr, const float *small, int64_t ld, int64_t rows, int64_t cols, int terms);

extern int g_bn_override;
extern int g_chunk_kb;
extern int g_pair_mode;
extern int g_persist_pairs;
extern int g_stream_k;
int gemm_pair_recover(cudaStream_t stream);
bool gemm_pair_eligible(const GemmParams &p, int bn, int a_mn, int b_mn, int terms);
int gemm_pair_launch(const float *A, const float *A_small, int64_t lda, int a_mn, const float *B, const float *B_small,
                     int64_t ldb, int b_mn, const GemmParams &p, int terms, cudaStream_t stream);
extern int g_split_k;

int gemm_tc_launch(const float *A, const float *A_small, int64_t lda, int a_mn, const float *B, const float *B_small,
                   int64_t ldb, int b_mn, const GemmParams &p, int terms, int bn_hint, cudaStream_t stream);

// Column sums of a GEMM epilogue (kEpiColsum): scratch for the per-slab partial sums (nullptr on allocation failure) and
// the pass that adds them, in a fixed order, to colsum[0..n_cols).
float *colsum_partial_scratch(int slabs, int64_t pitch);
int colsum_finish_launch(const float *partial, int slabs, int64_t pitch, int n_cols, float *colsum, cudaStream_t stream);
int colsum_finish2_launch(const float *partial, int slabs, int64_t pitch, int n_a, float *out_a, int n_b, float *out_b,
                          cudaStream_t stream);
int split_launch(const float *src, int64_t ld_src, int rows, int cols, const float *aux, int64_t ld_aux, float *dst_big,
                 float *dst_small, int64_t ld_dst, float *colsum, cudaStream_t stream);

int gemm_dispatch(int transA, int transB, int64_t M, int64_t N, int64_t K, const float *A, const float *A_small,
                  int64_t lda, const float *B, const float *B_small, int64_t ldb, float *D, float *D_small, int64_t ldd,
                  const float *bias, const float *mask_src, int64_t ld_mask, float *colsum, int flags, int precision,
                  cudaStream_t stream, bool reset_arena, int ohw = 0, const float *scale = nullptr);

// Communicator of the data-parallel step (comm_nccl.cpp): NCCL bound at run time, error polling, host watchdog.
struct Comm;
int comm_create(const void *id_bytes, int rank, int world, Comm **out);
int comm_destroy(Comm *c);
int comm_world(const Comm *c);
int comm_rank(const Comm *c);
int comm_allreduce_sum(Comm *c, float *buf, int64_t count, cudaStream_t stream);
int comm_poll(Comm *c);
int comm_abort(Comm *c);
int comm_watch(Comm *c, int timeout_ms, int (*done)(void *), void *arg);

int relu_forward_launch(const float *x, float *y, float *y_small, int64_t n, cudaStream_t s);
int relu_backward_launch(const float *gy, const float *ref, float *gx, int64_t n, cudaStream_t s);
int add_bias_launch(const float *x, const float *b, float *y, int64_t M, int64_t N, cudaStream_t s);
int softmax_ce_launch(const float *logits, const int32_t *t32, const int64_t *t64, int64_t B, int64_t C, float *loss,
                      float *dlogits, float *row_loss_scratch, float grad_scale, cudaStream_t s);
int adam_launch(float *p, float *g, float *m, float *v, float *p_small, int64_t n, int t, float lr, float b1, float b2,
                float eps, float hook_wd, float grad_scale, cudaStream_t s);
int sgd_launch(float *p, float *g, float *buf, float *p_small, int64_t n, float lr, float momentum, float wd,
               int nesterov, float hook_wd, float grad_scale, cudaStream_t s);
int conv_out_size(int64_t in, int k, int s, int p);
int im2col_launch(const float *x, float *col, float *col_small, int64_t N, int64_t C, int64_t H, int64_t W, int KH, int KW,
                  int S, int P, cudaStream_t s);
int col2im_launch(const float *col, int transposed, int64_t ld, float *gx, int64_t N, int64_t C, int64_t H, int64_t W,
                  int KH, int KW, int S, int P, cudaStream_t s);
int nchw_to_rows_launch(const float *src, float *dst, float *dst_small, int64_t N, int64_t OC, int64_t HW, int64_t ld,
                        cudaStream_t s);
int channel_sum_launch(const float *gy, float *gb, int64_t N, int64_t OC, int64_t HW, cudaStream_t s);

int linear_forward(const float *x, const float *x_small, const float *w, const float *w_small, const float *b, float *y,
                   float *y_small, int64_t M, int64_t N, int64_t K, int w_layout, int relu, int precision,
                   cudaStream_t stream);
int linear_backward(const float *x, const float *x_small, const float *w, const float *w_small, const float *dy, const float *dy_small,
                    const float *y, float *dx, float *dx_small, const float *dx_mask_src, float *dx_colsum, float *dw,
                    float *db, int64_t M, int64_t N, int64_t K, int w_layout, int precision, cudaStream_t stream,
                    cudaEvent_t dw_done = nullptr);
int conv2d_forward(const float *x, const float *w, const float *b, float *y, int64_t N, int64_t C, int64_t H, int64_t W,
                   int64_t OC, int KH, int KW, int S, int P, int act, int precision, cudaStream_t stream,
                   const float *scale = nullptr);
// Forward conv2d of small layers (OC <= 32, C*KH*KW <= 256) on the CUDA cores: see conv_fwd_direct.cu.
bool conv_fwd_direct_eligible(int64_t N, int64_t C, int64_t H, int64_t W, int64_t OC, int KH, int KW, int OH, int OW);
int conv_fwd_direct_launch(const float *x, const float *w, const float *bias, const float *scale, float *y, int64_t N,
                           int64_t C, int64_t H, int64_t W, int64_t OC, int KH, int KW, int S, int P, int OH, int OW, int act,
                           cudaStream_t stream);
bool conv_igemm_eligible(int64_t N, int64_t C, int64_t H, int64_t W, int64_t OC, int KH, int KW, int OH, int OW);
int conv_igemm_launch(const float *x, const float *w_big, const float *w_small, int64_t ldw, const float *bias,
                      const float *scale, float *y, int64_t N, int64_t C, int64_t H, int64_t W, int64_t OC, int KH, int KW,
                      int S, int P, int OH, int OW, int act, int terms, cudaStream_t stream);
// Input gradient of a stride-1 convolution through the same implicit GEMM (flipped, transposed weights).
bool conv_dx_igemm_eligible(int64_t N, int64_t C, int64_t H, int64_t W, int64_t OC, int KH, int KW, int S, int P, int OH,
                            int OW);
int conv_dx_igemm_launch(const float *gy, const float *w, float *wf, float *wf_small, float *gx, int64_t N, int64_t C,
                         int64_t H, int64_t W, int64_t OC, int KH, int KW, int P, int OH, int OW, int terms, cudaStream_t stream);
// D[m][n] = sum over z (ascending) of slices[z][m][n]; slices are [splits][M][lds].
int splitk_sum_launch(const float *slices, int splits, int M, int N, int lds, float *D, int ldd, cudaStream_t stream);
// Weight gradient through an implicit GEMM (no column matrix): see conv_dw_igemm.cu.
bool conv_dw_igemm_eligible(int64_t N, int64_t C, int64_t H, int64_t W, int64_t OC, int KH, int KW, int OH, int OW);
size_t conv_dw_igemm_scratch(int64_t N, int64_t C, int64_t OC, int KH, int KW, int OH, int OW);
int conv_dw_igemm_launch(const float *x, const float *gy, const float *gy_small, float *slices, float *gw, int64_t N,
                         int64_t C, int64_t H, int64_t W, int64_t OC, int KH, int KW, int S, int P, int OH, int OW, int terms,
                         cudaStream_t stream);
bool conv_dw_direct_eligible(int64_t N, int64_t C, int64_t H, int64_t W, int64_t OC, int KH, int KW, int OH, int OW);
int conv_dw_direct_launch(const float *x, const float *gy, float *gw, float *gb, int64_t N, int64_t C, int64_t H, int64_t W, int64_t OC,
                          int KH, int KW, int S, int P, int OH, int OW, int layout, cudaStream_t stream);
bool conv_dw_tile_eligible(int64_t N, int64_t C, int64_t H, int64_t W, int64_t OC, int KH, int KW, int S, int P, int OH, int OW);
int conv_dw_tile_launch(const float *x, const float *gy, float *gw, float *gb, int64_t N, int64_t C, int64_t H, int64_t W, int64_t OC,
                        int KH, int KW, int S, int P, int OH, int OW, int layout, cudaStream_t stream);
bool conv_dx_direct_eligible(int64_t N, int64_t C, int64_t H, int64_t W, int64_t OC, int KH, int KW, int S);
int conv_dx_direct_launch(const float *gy, const float *w, float *gx, int64_t N, int64_t C, int64_t H, int64_t W, int64_t OC,
                          int KH, int KW, int S, int P, int OH, int OW, int layout, cudaStream_t stream);
int conv2d_backward(const float *gy, const float *x, const float *w, float *gx, float *gw, float *gb, int64_t N, int64_t C,
                    int64_t H, int64_t W, int64_t OC, int KH, int KW, int S, int P, int mode, int precision,
                    cudaStream_t stream);

}  // namespace odl
