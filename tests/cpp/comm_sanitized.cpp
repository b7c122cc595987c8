// The communicator's host code (origindl_b200/csrc/comm_nccl.cpp: dlopen binding, error polling, watchdog, abort)
// compiled as ONE host program with AddressSanitizer and UndefinedBehaviorSanitizer, driven against the stand-in NCCL
// library (ODL_NCCL_LIBRARY).  No CUDA call is made: the translation unit only needs cudaStream_t as a type.  It walks
// the same scenarios as tests/test_comm_failure_detection.py -- create, poll, all-reduce, watchdog time-out with abort,
// refusal after abort, destroy -- so that a leak, a use after free (the aborted handle) or a bad cast shows up here.
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "../../origindl_b200/csrc/comm_nccl.cpp"

// the two functions of the library's error channel this translation unit calls (capi.cu provides them in the product)
namespace odl
{
static char g_err_text[1024];
void set_last_error(const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err_text, sizeof(g_err_text), fmt, ap);
    va_end(ap);
}
const char *get_last_error()
{
    return g_err_text;
}
}  // namespace odl

#define EXPECT(cond)                                                     \
    do                                                                   \
    {                                                                    \
        if (!(cond))                                                     \
        {                                                                \
            std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); \
            return 1;                                                    \
        }                                                                \
    } while (0)

int main()
{
    char token[ODL_COMM_UNIQUE_ID_BYTES];
    EXPECT(odl_comm_unique_id(token) == ODL_OK);
    void *comm = nullptr;
    EXPECT(odl_comm_create(token, 1, 4, &comm) == ODL_OK && comm);
    EXPECT(odl_comm_status(comm) == ODL_OK);
    float dummy[4] = {0, 0, 0, 0};
    EXPECT(odl_comm_allreduce(comm, dummy, 4, nullptr) == ODL_OK);
    EXPECT(odl_comm_allreduce(comm, nullptr, 4, nullptr) == ODL_ERR_INVALID_ARGUMENT);
    int calls = 0;
    auto soon = [](void *p) -> int { return ++*static_cast<int *>(p) >= 3; };
    EXPECT(odl_comm_watch(comm, 1000, soon, &calls) == ODL_OK && calls == 3);
    auto never = [](void *) -> int { return 0; };
    EXPECT(odl_comm_watch(comm, 50, never, nullptr) == ODL_ERR_COMM_TIMEOUT);
    EXPECT(std::strstr(odl::get_last_error(), "aborted") != nullptr);
    EXPECT(odl_comm_status(comm) == ODL_ERR_COMM);                       // refused: the handle is not touched again
    EXPECT(odl_comm_allreduce(comm, dummy, 4, nullptr) == ODL_ERR_COMM);
    EXPECT(odl_comm_destroy(comm) == ODL_OK);
    EXPECT(odl_comm_create(token, 4, 4, &comm) == ODL_ERR_INVALID_ARGUMENT);
    EXPECT(odl_comm_destroy(nullptr) == ODL_OK);
    std::printf("sanitized communicator run ok\n");
    return 0;
}
