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

struct alignas(64) TmapPack
{
    CUtensorMap a, a_small, b, b_small;
};

}  // namespace odl
