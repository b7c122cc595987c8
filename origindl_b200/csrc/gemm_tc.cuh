// Shared declarations for the tcgen05 GEMM: parameter block, epilogue flags, status codes.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace odl
{

// Status codes returned through the C ABI (0 = success).
enum Status : int
{
    kOk              = 0,
    kInvalidArgument = 1,   // null pointer, non-positive size, bad enum
    kMisaligned      = 2,   // pointer or leading dimension violates the 16-byte rule of the tiled loads
    kCudaError       = 3,   // a CUDA runtime / driver call failed (see odl_last_error)
    kKernelTimeout   = 4,   // a bounded wait inside a kernel ran out (device error flag was set)
    kTooLarge        = 5,   // size exceeds what the entry point supports
    kNotInitialized  = 6,
    kCommError       = 8,   // the communicator (NCCL) reported an error, is unavailable, or was aborted earlier
    kCommTimeout     = 9,   // a collective did not complete within the watchdog's limit; the communicator was aborted
    kStaleGraph      = 7,   // a recorded graph holds scratch addresses that have since been replaced: record it again
};

// Epilogue flags (bit set).  Order of application on each accumulator value v at (m, n):
//   v += bias[n]            (kEpiBias)
//   v  = v > 0 ? v : 0      (kEpiRelu)
//   v  = aux[m,n] > 0 ? v:0 (kEpiMask)   -- ReLU backward with the forward OUTPUT (or pre-activation) as aux
//   colsum[slab][n] = sum of v over the 32 rows of slab m/32   (kEpiColsum) -- plain stores of per-slab partial
//                             sums; the launcher adds them up in slab order afterwards (same bits every run)
//   D[m,n] = v ; D_small[m,n] = tf32(v - trunc_tf32(v))   (kEpiSmall) -- low part for the 3xTF32 split
enum EpiFlags : int
{
    kEpiBias   = 1,
    kEpiRelu   = 2,
    kEpiMask   = 4,
    kEpiColsum = 8,
    kEpiSmall  = 16,
    kEpiNCHW   = 32,  // D is [M/ohw][N][ohw] (conv output): row m = img*ohw + r goes to D[(img*N + n)*ohw + r]
    kEpiSplitK = 64,  // split-K (set by the launcher): the CTAs of split z store their partial tile into slice z of a
                      // scratch D [splits][M][ldd]; a second pass adds the slices in order (same bits every run)
    kEpiScale  = 128,  // v *= scale[n] before the bias (folded evaluation-mode BatchNorm); kEpiNCHW stores only
    kEpiSilu   = 256,  // v = v / (1 + exp(-v)) after bias / ReLU; kEpiNCHW stores only
};

struct GemmParams
{
    float *D;
    float *D_small;
    const float *bias;
    const float *scale;  // kEpiScale: per-column factor
    const float *aux;
    float *colsum;     // kEpiColsum: [ceil(M/128)*4][ld_colsum] per-slab partial column sums (scratch)
    int ld_colsum;
    int *err;  // device int: non-zero once any CTA gave up on a wait
    int M, N, K;
    int ldd, ld_aux;
    int flags;
    int ohw;           // kEpiNCHW: pixels per image
    int kb_per_split;  // K-blocks (of 32) handled by one CTA along gridDim.y; >= ceil(K/32) when not split
};

// The value the tensor core sees when it reads an fp32 container as tf32: low 13 mantissa bits dropped.
__host__ __device__ __forceinline__ float tf32_trunc(float x)
{
#ifdef __CUDA_ARCH__
    return __uint_as_float(__float_as_uint(x) & 0xffffe000u);
#else
    union
    {
        float f;
        uint32_t u;
    } c;
    c.f = x;
    c.u &= 0xffffe000u;
    return c.f;
#endif
}

#ifdef __CUDACC__
// Low part of the 3xTF32 split: x = trunc_tf32(x) + r exactly; r is then rounded to tf32 (round-to-nearest)
// so that the truncating read by the tensor core returns the rounded value itself.
__device__ __forceinline__ float tf32_small(float x)
{
    float r = x - tf32_trunc(x);
    uint32_t o;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(o) : "f"(r));
    return __uint_as_float(o);
}
#endif

}  // namespace odl
