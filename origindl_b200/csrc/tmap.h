// Tensor-map construction shared by the GEMM translation units.
#pragma once
#include <cuda.h>

#include <cstdint>

namespace odl
{

// Tensor map over a row-major fp32 matrix of `rows` x `cols` (row pitch `ld` elements) with a {box_cols, box_rows}
// tile.  Out-of-range parts of a tile are filled with zeros.  Returns a Status.
int make_tmap(CUtensorMap *out, const float *ptr, int64_t rows, int64_t cols, int64_t ld, int box_cols, int box_rows,
              CUtensorMapSwizzle swizzle);

// Tensor map for an MN-major operand: the row-major matrix [k_rows][mn_cols] (pitch ld) seen as the 3-D tensor
// {32 mn, k, mn / 32}, so that ONE copy moves `boxes` side-by-side 32 x box_k boxes (each 4 KB-aligned in shared memory,
// exactly where separate 2-D copies would put them).  mn_cols must be a multiple of 32.
int make_tmap_mn3d(CUtensorMap *out, const float *ptr, int64_t k_rows, int64_t mn_cols, int64_t ld, int box_k, int boxes,
                   CUtensorMapSwizzle swizzle);

struct alignas(64) TmapPack
{
    CUtensorMap a, a_small, b, b_small;
};

}  // namespace odl
