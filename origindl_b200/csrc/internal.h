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

extern int g_bn_override;
extern int g_chunk_kb;

int gemm_tc_launch(const float *A, const float *A_small, int64_t lda, int a_mn, const float *B, const float *B_small,
                   int64_t ldb, int b_mn, const GemmParams &p, int terms, int bn_hint, cudaStream_t stream);

int split_launch(const float *src, int64_t ld_src, int rows, int cols, const float *aux, int64_t ld_aux, float *dst_big,
                 float *dst_small, int64_t ld_dst, float *colsum, cudaStream_t stream);

int gemm_dispatch(int transA, int transB, int64_t M, int64_t N, int64_t K, const float *A, const float *A_small,
                  int64_t lda, const float *B, const float *B_small, int64_t ldb, float *D, float *D_small, int64_t ldd,
                  const float *bias, const float *mask_src, int64_t ld_mask, float *colsum, int flags, int precision,
                  cudaStream_t stream, bool reset_arena);

}  // namespace odl
