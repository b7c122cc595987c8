// A plain C++ host (no Python, no torch) running ONE rank of the data-parallel MLP step through the C ABI:
//     dp_two_ranks <rank> <world> <dir>        one process per GPU; rank 0 publishes NCCL's rendezvous token in <dir>
//     dp_two_ranks full <world> <dir>          the same global batch trained by one process alone (the yardstick)
// Every rank builds the same seeded parameters and the same seeded global batch, takes its rows, runs six
// odl_mlp_train_step_dp steps (backward with the overlapped per-layer all-reduce and the per-layer updates inside the
// library, layer 0's weight gradient in two row panels), checks each step with the watchdog, and writes its final
// parameters and per-step losses to <dir>.  tests/test_gpu_dp_cpp_host.py starts the processes and compares the files.
#include <cuda_runtime.h>

#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "odl_b200.h"

#define CHECK(expr)                                                                            \
    do                                                                                         \
    {                                                                                          \
        int _s = (expr);                                                                       \
        if (_s != ODL_OK)                                                                      \
        {                                                                                      \
            std::fprintf(stderr, "%s -> status %d: %s\n", #expr, _s, odl_last_error());        \
            return 1;                                                                          \
        }                                                                                      \
    } while (0)

static uint32_t g_state = 1;
static float next_uniform()  // [-1, 1), the same sequence in every process
{
    g_state = g_state * 1664525u + 1013904223u;
    return static_cast<float>(static_cast<int32_t>(g_state >> 8) % 65536) / 32768.0f - 1.0f;
}

static bool write_file(const std::string &path, const void *data, size_t bytes)
{
    const std::string tmp = path + ".tmp";
    FILE *f               = std::fopen(tmp.c_str(), "wb");
    if (!f)
        return false;
    const bool ok = std::fwrite(data, 1, bytes, f) == bytes;
    std::fclose(f);
    return ok && std::rename(tmp.c_str(), path.c_str()) == 0;  // readers never see a partial file
}

static bool read_file_when_present(const std::string &path, void *data, size_t bytes, int timeout_s)
{
    for (int i = 0; i < timeout_s * 20; ++i)
    {
        FILE *f = std::fopen(path.c_str(), "rb");
        if (f)
        {
            const bool ok = std::fread(data, 1, bytes, f) == bytes;
            std::fclose(f);
            if (ok)
                return true;
        }
        std::this_thread::sleep_for(std::chrono::milliseconds(50));
    }
    return false;
}

int main(int argc, char **argv)
{
    if (argc != 4)
    {
        std::fprintf(stderr, "usage: dp_two_ranks <rank|full> <world> <dir>\n");
        return 2;
    }
    const bool full       = std::string(argv[1]) == "full";
    const int world       = std::atoi(argv[2]);
    const int rank        = full ? 0 : std::atoi(argv[1]);
    const std::string dir = argv[3];
    const int32_t sizes[4] = {256, 384, 256, 10};
    const int per = 128, steps = 6, global = per * world;
    const int batch = full ? global : per;

    if (cudaSetDevice(rank) != cudaSuccess)
    {
        std::fprintf(stderr, "cudaSetDevice(%d) failed\n", rank);
        return 1;
    }
    CHECK(odl_init(rank));
    void *mlp = nullptr;
    CHECK(odl_mlp_create(sizes, 4, batch, /*Adam*/ 1, 1e-3f, 0.0f, 1e-4f, ODL_PRECISION_3XTF32, &mlp));

    // identical parameters everywhere: uniform(-sqrt(6 / in), +) weights, zero biases
    std::vector<float> params(static_cast<size_t>(odl_mlp_param_count(mlp)));
    size_t o = 0;
    for (int l = 0; l < 3; ++l)
    {
        const float bound = std::sqrt(6.0f / sizes[l]);
        for (int i = 0; i < sizes[l] * sizes[l + 1]; ++i)
            params[o++] = bound * next_uniform();
        for (int i = 0; i < sizes[l + 1]; ++i)
            params[o++] = 0.0f;
    }
    CHECK(odl_mlp_set_params(mlp, params.data(), nullptr));
    // two global batches, alternated; a rank uploads only its rows
    std::vector<float> x(2 * static_cast<size_t>(global) * sizes[0]);
    std::vector<int32_t> t(2 * static_cast<size_t>(global));
    for (auto &v : x)
        v = 2.0f * next_uniform();
    for (auto &v : t)
        v = static_cast<int32_t>((next_uniform() + 1.0f) * 0.5f * 10.0f) % 10;
    float *dx[2];
    int32_t *dt[2];
    for (int b = 0; b < 2; ++b)
    {
        const size_t row0 = static_cast<size_t>(b) * global + (full ? 0 : static_cast<size_t>(rank) * per);
        if (cudaMalloc(&dx[b], static_cast<size_t>(batch) * sizes[0] * 4) != cudaSuccess ||
            cudaMalloc(&dt[b], static_cast<size_t>(batch) * 4) != cudaSuccess)
            return 1;
        cudaMemcpy(dx[b], x.data() + row0 * sizes[0], static_cast<size_t>(batch) * sizes[0] * 4, cudaMemcpyHostToDevice);
        cudaMemcpy(dt[b], t.data() + row0, static_cast<size_t>(batch) * 4, cudaMemcpyHostToDevice);
    }

    void *comm = nullptr;
    if (!full)
    {
        char token[ODL_COMM_UNIQUE_ID_BYTES];
        if (rank == 0)
        {
            CHECK(odl_comm_unique_id(token));
            if (!write_file(dir + "/token", token, sizeof(token)))
                return 1;
        }
        else if (!read_file_when_present(dir + "/token", token, sizeof(token), 60))
        {
            std::fprintf(stderr, "rank %d: no rendezvous token within 60 s\n", rank);
            return 1;
        }
        CHECK(odl_comm_create(token, rank, world, &comm));
        CHECK(odl_mlp_dp_attach(mlp, comm, 2));
    }
    std::vector<float> losses(steps);
    for (int s = 0; s < steps; ++s)
    {
        if (full)
            CHECK(odl_mlp_train_step(mlp, dx[s & 1], dt[s & 1], 0, nullptr));
        else
        {
            CHECK(odl_mlp_train_step_dp(mlp, dx[s & 1], dt[s & 1], 0, nullptr));
            CHECK(odl_mlp_dp_wait(mlp, 30000));  // watchdog: the step's last all-reduce completed, no asynchronous error
            CHECK(odl_comm_status(comm));
        }
        CHECK(odl_device_status(nullptr));
        cudaMemcpy(&losses[s], odl_mlp_loss_ptr(mlp), 4, cudaMemcpyDeviceToHost);
    }
    CHECK(odl_mlp_get_packed(mlp, 0, params.data(), nullptr));
    const std::string tag = full ? "full" : std::to_string(rank);
    if (!write_file(dir + "/params_" + tag + ".bin", params.data(), params.size() * 4) ||
        !write_file(dir + "/losses_" + tag + ".bin", losses.data(), losses.size() * 4))
        return 1;
    CHECK(odl_mlp_destroy(mlp));
    if (comm)
        CHECK(odl_comm_destroy(comm));
    std::printf("%s done: loss %.6f -> %.6f\n", tag.c_str(), losses.front(), losses.back());
    return 0;
}
