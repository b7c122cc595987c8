/* Stand-in for libnccl.so.2, for CPU tests of the communicator's failure handling (origindl_b200/csrc/comm_nccl.cpp).
 *
 * It exports the handful of NCCL entry points the library binds and moves no data; a test tells it, through the
 * fake_nccl_* setters below, to report an asynchronous error after a number of polls or to fail an initialisation,
 * and reads back how often the communicator was aborted.  Loaded through ODL_NCCL_LIBRARY, never on a GPU box's
 * data path.  Result codes follow NCCL's public enumeration (0 success, 2 system error, 6 remote error, 7 in progress). */
#include <stddef.h>
#include <stdlib.h>
#include <string.h>

typedef struct
{
    char internal[128];
} FakeUniqueId;

typedef struct
{
    int rank, world, polls, aborted;
} FakeComm;

static int g_init_error   = 0;
static int g_async_after  = -1; /* polls before the asynchronous error shows; < 0: never */
static int g_async_error  = 0;
static int g_abort_count  = 0;
static int g_reduce_count = 0;
static int g_live_comms   = 0;

void fake_nccl_set_init_error(int code) { g_init_error = code; }
void fake_nccl_set_async_error(int after_polls, int code) { g_async_after = after_polls, g_async_error = code; }
int fake_nccl_abort_count(void) { return g_abort_count; }
int fake_nccl_allreduce_count(void) { return g_reduce_count; }
int fake_nccl_live_comms(void) { return g_live_comms; }

int ncclGetVersion(int *v)
{
    *v = 0;
    return 0;
}

int ncclGetUniqueId(FakeUniqueId *id)
{
    memset(id->internal, 0, sizeof(id->internal));
    memcpy(id->internal, "fake-nccl-id", 12);
    return 0;
}

int ncclCommInitRank(void **comm, int world, FakeUniqueId id, int rank)
{
    if (g_init_error)
        return g_init_error;
    if (memcmp(id.internal, "fake-nccl-id", 12) != 0)
        return 4; /* invalid argument: the token did not come from ncclGetUniqueId */
    FakeComm *c = (FakeComm *)calloc(1, sizeof(FakeComm));
    c->rank = rank, c->world = world;
    *comm = c;
    ++g_live_comms;
    return 0;
}

int ncclCommDestroy(void *comm)
{
    free(comm);
    --g_live_comms;
    return 0;
}

int ncclCommAbort(void *comm)
{
    ++g_abort_count;
    free(comm);
    --g_live_comms;
    return 0;
}

int ncclCommGetAsyncError(void *comm, int *async_error)
{
    FakeComm *c  = (FakeComm *)comm;
    *async_error = (g_async_after >= 0 && c->polls >= g_async_after) ? g_async_error : 0;
    ++c->polls;
    return 0;
}

int ncclAllReduce(const void *send, void *recv, size_t count, int dtype, int op, void *comm, void *stream)
{
    (void)send, (void)recv, (void)count, (void)dtype, (void)op, (void)comm, (void)stream;
    ++g_reduce_count;
    return 0;
}

const char *ncclGetErrorString(int code)
{
    switch (code)
    {
        case 0: return "no error";
        case 2: return "unhandled system error";
        case 6: return "remote process exited or there was a network error";
        case 7: return "in progress";
        default: return "fake nccl error";
    }
}
