// NVTX ranges around the phases of a training step (forward, loss, backward of layer l, all-reduce of bucket l,
// optimizer), for timeline tools.  Off unless the environment variable ODL_NVTX is set to a non-zero value, so that a
// production run pays one predictable branch per phase.  NVTX v3 is header-only: without an attached tool the calls
// fall through a null function table.  The reference has no tracing hooks of any kind.
#pragma once
#include <nvtx3/nvToolsExt.h>

#include <cstdio>
#include <cstdlib>

namespace odl
{

inline bool nvtx_enabled()
{
    static const bool on = [] {
        const char *v = std::getenv("ODL_NVTX");
        return v && *v && *v != '0';
    }();
    return on;
}

// Number of ranges opened so far in this process (tests read it to see that the switch works without a profiler).
inline long long &nvtx_range_count()
{
    static long long n = 0;
    return n;
}

struct NvtxRange
{
    bool open;
    explicit NvtxRange(const char *name, int index = -1) : open(nvtx_enabled())
    {
        if (!open)
            return;
        char buf[64];
        if (index >= 0)
        {
            std::snprintf(buf, sizeof(buf), "%s %d", name, index);
            name = buf;
        }
        nvtxRangePushA(name);
        ++nvtx_range_count();
    }
    ~NvtxRange()
    {
        if (open)
            nvtxRangePop();
    }
    NvtxRange(const NvtxRange &)            = delete;
    NvtxRange &operator=(const NvtxRange &) = delete;
};

}  // namespace odl
