// Communicator of the data-parallel step: NCCL all-reduce over NVLink / NVSwitch, bound at run time.
//
// The reference has no multi-GPU layer at all (no collective, no stream, no peer copy anywhere in its tree); this is
// the new piece the data-parallel MLP step needs: one communicator per process (or thread) and GPU, gradients summed in
// place in the flat gradient buffer.  NCCL is resolved with dlopen so that the library links against nothing but the
// CUDA runtime: inside a torch process "libnccl.so.2" is the copy torch already loaded, a plain C++ host points
// ODL_NCCL_LIBRARY at the one it wants.  Only NCCL's public C interface is used.
//
// Failure detection (the counterpart of the reference's CUDA_CHECK_ASYNC, include/origin/mat/origin/cuda/cuda_utils.cuh:14-33,
// for the one thing that can stall without a CUDA error: a peer that never joins a collective):
//   * comm_poll        asks NCCL for errors it noticed asynchronously (ncclCommGetAsyncError) and maps them to a status;
//   * comm_watch       a host watchdog: polls a caller-supplied "is the step's last collective done" query and comm_poll
//                      until done, error or time-out; on error or time-out it aborts the communicator (ncclCommAbort ends
//                      kernels that wait for the missing peer, so the GPU and the context stay usable) and returns
//                      kCommError / kCommTimeout.  An aborted communicator refuses every later call.
// Both are exercised on the CPU against a stand-in NCCL library that misbehaves on request (tests/cpp/fake_nccl.c).
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <chrono>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>

#include "../../include/odl_b200.h"
#include "gemm_tc.cuh"
#include "host_util.h"
#include "internal.h"

namespace odl
{

namespace
{
// The slice of NCCL's public C interface used here.
struct NcclUniqueId
{
    char internal[ODL_COMM_UNIQUE_ID_BYTES];
};
using NcclComm                  = void *;
constexpr int kNcclSuccess      = 0;
constexpr int kNcclInProgress   = 7;
constexpr int kNcclFloat32      = 7;
constexpr int kNcclSum          = 0;

struct NcclApi
{
    void *lib = nullptr;
    std::string path, error;
    int (*GetVersion)(int *)                                                                       = nullptr;
    int (*GetUniqueId)(NcclUniqueId *)                                                             = nullptr;
    int (*CommInitRank)(NcclComm *, int, NcclUniqueId, int)                                        = nullptr;
    int (*CommDestroy)(NcclComm)                                                                   = nullptr;
    int (*CommAbort)(NcclComm)                                                                     = nullptr;
    int (*CommGetAsyncError)(NcclComm, int *)                                                      = nullptr;
    int (*AllReduce)(const void *, void *, size_t, int, int, NcclComm, cudaStream_t)               = nullptr;
    const char *(*GetErrorString)(int)                                                             = nullptr;
};

NcclApi g_api;
std::once_flag g_api_once;

template <typename F>
bool bind(void *lib, const char *name, F *out, std::string *err)
{
    *out = reinterpret_cast<F>(dlsym(lib, name));
    if (!*out)
        *err = std::string("symbol ") + name + " not found";
    return *out != nullptr;
}

const NcclApi &nccl()
{
    std::call_once(g_api_once, [] {
        const char *env = std::getenv("ODL_NCCL_LIBRARY");
        const char *candidates[3] = {env, "libnccl.so.2", "libnccl.so"};
        for (const char *c : candidates)
        {
            if (!c || !*c)
                continue;
            g_api.lib = dlopen(c, RTLD_NOW | RTLD_GLOBAL);
            if (g_api.lib)
            {
                g_api.path = c;
                break;
            }
            g_api.error = dlerror();
            if (c == env)
                break;  // an explicit choice that does not load is an error, not a reason to pick another library
        }
        if (!g_api.lib)
            return;
        std::string e;
        bool ok = bind(g_api.lib, "ncclGetUniqueId", &g_api.GetUniqueId, &e) &&
                  bind(g_api.lib, "ncclCommInitRank", &g_api.CommInitRank, &e) &&
                  bind(g_api.lib, "ncclCommDestroy", &g_api.CommDestroy, &e) &&
                  bind(g_api.lib, "ncclCommAbort", &g_api.CommAbort, &e) &&
                  bind(g_api.lib, "ncclCommGetAsyncError", &g_api.CommGetAsyncError, &e) &&
                  bind(g_api.lib, "ncclAllReduce", &g_api.AllReduce, &e) &&
                  bind(g_api.lib, "ncclGetErrorString", &g_api.GetErrorString, &e);
        bind(g_api.lib, "ncclGetVersion", &g_api.GetVersion, &e);  // optional
        if (!ok)
        {
            g_api.error = g_api.path + ": " + e;
            g_api.lib   = nullptr;
        }
    });
    return g_api;
}

int need_api(const NcclApi **out)
{
    const NcclApi &a = nccl();
    if (!a.lib)
    {
        set_last_error("NCCL is not available (%s); set ODL_NCCL_LIBRARY to the libnccl.so.2 to use",
                       a.error.empty() ? "library not found" : a.error.c_str());
        return kCommError;
    }
    *out = &a;
    return kOk;
}
}  // namespace

struct Comm
{
    NcclComm handle = nullptr;
    int rank = 0, world = 1;
    bool aborted = false;
    std::mutex mu;
};

namespace
{
int nccl_fail(const NcclApi &a, const char *what, int code)
{
    set_last_error("%s failed: NCCL error %d (%s)", what, code, a.GetErrorString ? a.GetErrorString(code) : "?");
    return kCommError;
}

int usable(Comm *c)
{
    if (!c || !c->handle)
    {
        set_last_error("communicator: null handle");
        return kInvalidArgument;
    }
    if (c->aborted)
    {
        set_last_error("communicator was aborted after a failure; create a new one");
        return kCommError;
    }
    return kOk;
}
}  // namespace

int comm_create(const void *id_bytes, int rank, int world, Comm **out)
{
    if (!id_bytes || !out || world < 1 || rank < 0 || rank >= world)
    {
        set_last_error("comm_create: invalid argument (rank %d of %d)", rank, world);
        return kInvalidArgument;
    }
    const NcclApi *a;
    int rc = need_api(&a);
    if (rc)
        return rc;
    NcclUniqueId id;
    std::memcpy(&id, id_bytes, sizeof(id));
    NcclComm h = nullptr;
    int e      = a->CommInitRank(&h, world, id, rank);
    if (e != kNcclSuccess || !h)
        return nccl_fail(*a, "ncclCommInitRank", e);
    Comm *c   = new Comm();
    c->handle = h, c->rank = rank, c->world = world;
    *out      = c;
    return kOk;
}

int comm_destroy(Comm *c)
{
    if (!c)
        return kOk;
    const NcclApi &a = nccl();
    if (a.lib && c->handle)
    {
        if (c->aborted)
            ;  // ncclCommAbort already released it
        else
            a.CommDestroy(c->handle);
    }
    delete c;
    return kOk;
}

int comm_world(const Comm *c)
{
    return c ? c->world : 1;
}

int comm_rank(const Comm *c)
{
    return c ? c->rank : 0;
}

// In-place sum of `count` floats over all ranks, enqueued on `stream`.
int comm_allreduce_sum(Comm *c, float *buf, int64_t count, cudaStream_t stream)
{
    int rc = usable(c);
    if (rc)
        return rc;
    if (!buf || count <= 0)
    {
        set_last_error("comm_allreduce: invalid argument (count=%lld)", (long long)count);
        return kInvalidArgument;
    }
    const NcclApi &a = nccl();
    int e = a.AllReduce(buf, buf, static_cast<size_t>(count), kNcclFloat32, kNcclSum, c->handle, stream);
    if (e != kNcclSuccess)
        return nccl_fail(a, "ncclAllReduce", e);
    return kOk;
}

// Errors NCCL noticed on its own threads since the last call (a peer that died, a failed transport).
int comm_poll(Comm *c)
{
    int rc = usable(c);
    if (rc)
        return rc;
    const NcclApi &a = nccl();
    int async        = kNcclSuccess;
    int e            = a.CommGetAsyncError(c->handle, &async);
    if (e != kNcclSuccess)
        return nccl_fail(a, "ncclCommGetAsyncError", e);
    if (async != kNcclSuccess && async != kNcclInProgress)
    {
        set_last_error("communicator reports an asynchronous error: NCCL error %d (%s)", async,
                       a.GetErrorString ? a.GetErrorString(async) : "?");
        return kCommError;
    }
    return kOk;
}

int comm_abort(Comm *c)
{
    if (!c || !c->handle || c->aborted)
        return kOk;
    std::lock_guard<std::mutex> lk(c->mu);
    if (c->aborted)
        return kOk;
    const NcclApi &a = nccl();
    if (a.lib)
        a.CommAbort(c->handle);
    c->aborted = true;
    return kOk;
}

// Host watchdog.  done(arg) returns non-zero once the work being watched has completed.  On an asynchronous error or
// after timeout_ms the communicator is aborted: collectives still waiting for a peer end, later calls are refused.
int comm_watch(Comm *c, int timeout_ms, int (*done)(void *), void *arg)
{
    int rc = usable(c);
    if (rc)
        return rc;
    if (!done || timeout_ms < 0)
    {
        set_last_error("comm_watch: invalid argument");
        return kInvalidArgument;
    }
    const auto t0 = std::chrono::steady_clock::now();
    for (unsigned spin = 0;; ++spin)
    {
        if (done(arg))
            return comm_poll(c);
        if ((rc = comm_poll(c)))
        {
            const std::string msg = get_last_error();
            comm_abort(c);
            set_last_error("%s; communicator aborted", msg.c_str());
            return rc;
        }
        const auto waited = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
        if (waited >= timeout_ms)
        {
            comm_abort(c);
            set_last_error("collective did not complete within %d ms (a peer never joined?); communicator aborted", timeout_ms);
            return kCommTimeout;
        }
        if (spin < 64)
            std::this_thread::yield();
        else
            std::this_thread::sleep_for(std::chrono::microseconds(200));
    }
}

}  // namespace odl

using namespace odl;

extern "C" {

int odl_comm_unique_id(void *id_bytes)
{
    if (!id_bytes)
    {
        set_last_error("comm_unique_id: null pointer");
        return kInvalidArgument;
    }
    const NcclApi *a;
    int rc = need_api(&a);
    if (rc)
        return rc;
    NcclUniqueId id;
    int e = a->GetUniqueId(&id);
    if (e != kNcclSuccess)
        return nccl_fail(*a, "ncclGetUniqueId", e);
    std::memcpy(id_bytes, &id, sizeof(id));
    return kOk;
}

int odl_comm_create(const void *id_bytes, int rank, int world, void **comm)
{
    Comm *c = nullptr;
    int rc  = comm_create(id_bytes, rank, world, &c);
    if (rc == kOk)
        *comm = c;
    return rc;
}

int odl_comm_destroy(void *comm)
{
    return comm_destroy(static_cast<Comm *>(comm));
}

int odl_comm_allreduce(void *comm, float *buf, int64_t count, void *stream)
{
    return comm_allreduce_sum(static_cast<Comm *>(comm), buf, count, static_cast<cudaStream_t>(stream));
}

int odl_comm_status(void *comm)
{
    return comm_poll(static_cast<Comm *>(comm));
}

int odl_comm_watch(void *comm, int timeout_ms, int (*done)(void *), void *arg)
{
    return comm_watch(static_cast<Comm *>(comm), timeout_ms, done, arg);
}

}  // extern "C"
