// Batch assembly on the device: dst[i, :] = src[idx[i], :] and labels_dst[i] = labels_src[idx[i]] in one launch.
//
// The reference's DataLoader::next (src/data/dataloader.cpp:38-139) builds every batch on the host, sample by sample
// (get_item -> to_vector -> push_back -> one flat vector -> Tensor), and the training loop then moves it to the
// device.  With 180 GB of HBM the whole training set of the reference's examples stays resident on the GPU, so a batch
// is a row gather driven by the (shuffled) index list: the only host-to-device traffic per step is the indices.
//
// HBM-bound: one warp per output row, float4 loads and stores when the row pitch allows it, grid sized in multiples of
// the SM count.  An index outside [0, n_src) raises the device error flag (code 3) and writes zeros / label -1 instead
// of reading out of bounds.
#include <cuda_runtime.h>

#include "../../include/odl_b200.h"
#include "gemm_tc.cuh"
#include "host_util.h"
#include "internal.h"

namespace odl
{
namespace
{
__global__ void __launch_bounds__(256) gather_rows_kernel(const float *__restrict__ src, int64_t ld_src, int64_t n_src,
                                                          const int64_t *__restrict__ idx, int64_t n_idx, int64_t cols,
                                                          float *__restrict__ dst, int64_t ld_dst,
                                                          const int64_t *__restrict__ labels_src,
                                                          int64_t *__restrict__ labels_dst, int vec4, int *__restrict__ err)
{
    const int lane        = threadIdx.x & 31;
    const int64_t warp0   = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t n_warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
    for (int64_t r = warp0; r < n_idx; r += n_warps)
    {
        const int64_t s = idx[r];
        const bool ok   = s >= 0 && s < n_src;
        if (!ok && lane == 0)
            if (err)
                atomicExch(err, 3);
        if (labels_dst && lane == 0)
            labels_dst[r] = ok ? labels_src[s] : -1;
        float *out = dst + r * ld_dst;
        if (vec4)
        {
            const float4 *in4 = reinterpret_cast<const float4 *>(src + (ok ? s : 0) * ld_src);
            float4 *out4      = reinterpret_cast<float4 *>(out);
            const int64_t q   = cols >> 2;
            for (int64_t c = lane; c < q; c += 32)
                out4[c] = ok ? __ldg(in4 + c) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        else
        {
            const float *in = src + (ok ? s : 0) * ld_src;
            for (int64_t c = lane; c < cols; c += 32)
                out[c] = ok ? __ldg(in + c) : 0.f;
        }
    }
}
}  // namespace
}  // namespace odl

using namespace odl;

extern "C" int odl_gather_rows(const float *src, int64_t ld_src, int64_t n_src, const int64_t *idx, int64_t n_idx,
                               int64_t cols, float *dst, int64_t ld_dst, const int64_t *labels_src, int64_t *labels_dst,
                               void *stream)
{
    if (!is_ready())
    {
        // the kernel reports an out-of-range index through the per-device flag odl_init allocates
        set_last_error("odl_init has not been called");
        return kNotInitialized;
    }
    if (!src || !idx || !dst || n_src <= 0 || n_idx <= 0 || cols <= 0 || ld_src < cols || ld_dst < cols ||
        (labels_dst && !labels_src))
    {
        set_last_error("gather_rows: invalid argument (n_src=%lld n_idx=%lld cols=%lld ld_src=%lld ld_dst=%lld)",
                       (long long)n_src, (long long)n_idx, (long long)cols, (long long)ld_src, (long long)ld_dst);
        return kInvalidArgument;
    }
    const bool vec4 = !(cols & 3) && !(ld_src & 3) && !(ld_dst & 3) && !(reinterpret_cast<uintptr_t>(src) & 15) &&
                      !(reinterpret_cast<uintptr_t>(dst) & 15);
    int64_t blocks = (n_idx + 7) / 8;  // 8 warps per block, one row per warp and pass
    if (blocks > 148 * 8)
        blocks = 148 * 8;
    gather_rows_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        src, ld_src, n_src, idx, n_idx, cols, dst, ld_dst, labels_src, labels_dst, vec4 ? 1 : 0, device_error_flag());
    ++g_launch_count;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
    {
        set_last_error("gather_rows_kernel launch failed: %s", cudaGetErrorString(e));
        return kCudaError;
    }
    return kOk;
}
