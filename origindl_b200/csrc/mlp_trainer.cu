// Device-resident MLP training state behind the C ABI: the fused equivalent of
//   nn::MLP::forward (src/nn/models/mlp.cpp:43-61)  ->  functional::softmax_cross_entropy
//   -> Tensor::backward (src/core/tensor_impl.cpp:78-278)  ->  Optimizer::step (src/optim/optimizer.cpp:19-53)
// of the reference, with every tensor of the step living in buffers allocated once:
//   * one flat parameter buffer [W_0 {in,out}, b_0, W_1, b_1, ...] (segments padded to 64 floats) with matching
//     flat buffers for the low TF32 parts, the gradients and the optimizer moments, so the optimizer is ONE launch
//     and a layer's gradient bucket [dW_l, db_l] is one contiguous range for the all-reduce;
//   * per-layer activations y_l (+ low parts, written by the forward GEMM's epilogue) and two ping-pong buffers for
//     the back-propagated gradient (+ low parts, written by the dX GEMM's epilogue together with the ReLU mask and
//     the bias gradient of the layer below).
// Per step: 1 split of the input, L forward GEMMs, 2 loss launches, 1 split of dlogits, 2L-1 backward GEMMs, 1 optimizer.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "../../include/odl_b200.h"
#include "gemm_tc.cuh"
#include "host_util.h"
#include "internal.h"
#include "nvtx_ranges.h"

namespace odl
{

namespace
{
inline int64_t pad64(int64_t x)
{
    return (x + 63) & ~int64_t(63);
}

struct Mlp
{
    std::vector<int> sizes;
    int L          = 0;
    int64_t batch  = 0;
    int optimizer  = 1;  // 0 SGD, 1 Adam
    float lr = 1e-3f, momentum = 0.f, hook_wd = 0.f;
    float beta1 = 0.9f, beta2 = 0.999f, eps = 1e-8f;
    int precision  = ODL_PRECISION_3XTF32;
    int step_count = 0;
    std::vector<int64_t> w_off, b_off;  // offsets (floats) into the flat buffers
    int64_t total = 0;
    float *params = nullptr, *params_small = nullptr, *grads = nullptr, *m = nullptr, *v = nullptr;
    float *x_small = nullptr;
    std::vector<float *> act, act_small;  // y_l, l = 0..L-1 (act[L-1] = logits)
    float *gbuf[2] = {nullptr, nullptr}, *gbuf_small[2] = {nullptr, nullptr};
    float *row_loss = nullptr, *loss = nullptr;
    const float *cur_x = nullptr;
    int64_t max_width = 0;
    std::vector<void *> allocs;
    cudaGraphExec_t step_graph = nullptr;  // forward + loss + backward of one step on fixed input buffers (odl_mlp_capture)
    long long graph_launches   = 0;        // kernels one replay of it runs
    // data-parallel step (odl_mlp_dp_attach): communicator (not owned), its stream, and per gradient piece one event
    // "gradients final" (compute stream) and one "reduced" (communication stream).  Pieces: layers L-1 ... 1, then the
    // dw0_panels row panels of layer 0.
    Comm *comm               = nullptr;
    cudaStream_t comm_stream = nullptr;
    int dw0_panels           = 1;
    std::vector<cudaEvent_t> ev_ready, ev_reduced;
    cudaEvent_t ev_step_done = nullptr;    // the communication stream has finished the step (last reduction and update)
    long long graph_generation = -1;       // scratch_generation() when it was recorded: its scratch addresses are valid
                                           // only while no scratch block has been replaced since
    // ev_layer_done[l]: layer l's backward (its dX GEMM, the last reader of W_l) is complete on the compute stream -- what
    // layer l's update on the communication stream waits for
    std::vector<cudaEvent_t> ev_layer_done;

    template <typename T>
    int alloc(T **p, size_t count)
    {
        void *q       = nullptr;
        cudaError_t e = cudaMalloc(&q, count * sizeof(T));
        if (e != cudaSuccess)
        {
            set_last_error("mlp: cudaMalloc(%zu) failed: %s", count * sizeof(T), cudaGetErrorString(e));
            return kCudaError;
        }
        allocs.push_back(q);
        *p = static_cast<T *>(q);
        return kOk;
    }
    void drop_dp()
    {
        for (cudaEvent_t e : ev_ready)
            cudaEventDestroy(e);
        for (cudaEvent_t e : ev_reduced)
            cudaEventDestroy(e);
        for (cudaEvent_t e : ev_layer_done)
            cudaEventDestroy(e);
        ev_ready.clear(), ev_reduced.clear(), ev_layer_done.clear();
        if (ev_step_done)
            cudaEventDestroy(ev_step_done);
        ev_step_done = nullptr;
        if (comm_stream)
            cudaStreamDestroy(comm_stream);
        comm_stream = nullptr;
        comm        = nullptr;
    }
    ~Mlp()
    {
        drop_dp();
        if (step_graph)
            cudaGraphExecDestroy(step_graph);
        for (void *q : allocs)
            cudaFree(q);
    }
};

inline bool three(const Mlp *h)
{
    return h->precision == ODL_PRECISION_3XTF32;
}
}  // namespace
}  // namespace odl

using namespace odl;
#define ST(x) static_cast<cudaStream_t>(x)
#define H(x) static_cast<Mlp *>(x)

extern "C" {

int odl_mlp_create(const int32_t *sizes, int n_sizes, int64_t batch, int optimizer, float lr, float momentum,
                   float hook_weight_decay, int precision, void **handle)
{
    if (!is_ready())
    {
        set_last_error("odl_init has not been called");
        return kNotInitialized;
    }
    if (!sizes || n_sizes < 2 || batch <= 0 || !handle || (optimizer != 0 && optimizer != 1))
    {
        set_last_error("MLP requires at least 2 layer sizes (input and output), but got %d", n_sizes);
        return kInvalidArgument;
    }
    Mlp *h       = new Mlp();
    h->sizes.assign(sizes, sizes + n_sizes);
    h->L         = n_sizes - 1;
    h->batch     = batch;
    h->optimizer = optimizer;
    h->lr = lr, h->momentum = momentum, h->hook_wd = hook_weight_decay, h->precision = precision;
    int64_t off = 0;
    for (int l = 0; l < h->L; ++l)
    {
        if (sizes[l] <= 0 || sizes[l + 1] <= 0)
        {
            delete h;
            set_last_error("mlp: layer sizes must be positive");
            return kInvalidArgument;
        }
        h->w_off.push_back(off);
        off += pad64(static_cast<int64_t>(sizes[l]) * sizes[l + 1]);
        h->b_off.push_back(off);
        off += pad64(sizes[l + 1]);
        if (sizes[l + 1] > h->max_width)
            h->max_width = sizes[l + 1];
    }
    h->total = off;
    int rc   = 0;
    rc |= h->alloc(&h->params, off);
    rc |= h->alloc(&h->grads, off);
    rc |= h->alloc(&h->m, off);  // Adam first moment / SGD momentum buffer
    if (optimizer == 1)
        rc |= h->alloc(&h->v, off);
    if (three(h))
    {
        rc |= h->alloc(&h->params_small, off);
        rc |= h->alloc(&h->x_small, static_cast<size_t>(batch) * sizes[0]);
    }
    h->act.resize(h->L, nullptr);
    h->act_small.resize(h->L, nullptr);
    for (int l = 0; l < h->L && !rc; ++l)
    {
        rc |= h->alloc(&h->act[l], static_cast<size_t>(batch) * sizes[l + 1]);
        if (three(h) && l + 1 < h->L)
            rc |= h->alloc(&h->act_small[l], static_cast<size_t>(batch) * sizes[l + 1]);
    }
    for (int i = 0; i < 2 && !rc; ++i)
    {
        rc |= h->alloc(&h->gbuf[i], static_cast<size_t>(batch) * h->max_width);
        if (three(h))
            rc |= h->alloc(&h->gbuf_small[i], static_cast<size_t>(batch) * h->max_width);
    }
    rc |= h->alloc(&h->row_loss, static_cast<size_t>(batch));
    rc |= h->alloc(&h->loss, 1);
    if (rc)
    {
        delete h;
        return kCudaError;
    }
    cudaMemset(h->params, 0, off * 4);
    cudaMemset(h->grads, 0, off * 4);
    cudaMemset(h->m, 0, off * 4);
    if (h->v)
        cudaMemset(h->v, 0, off * 4);
    if (h->params_small)
        cudaMemset(h->params_small, 0, off * 4);
    *handle = h;
    return kOk;
}

int odl_mlp_destroy(void *handle)
{
    cudaDeviceSynchronize();
    delete H(handle);
    return kOk;
}

int64_t odl_mlp_param_count(void *handle)
{
    int64_t n = 0;
    Mlp *h    = H(handle);
    for (int l = 0; l < h->L; ++l)
        n += static_cast<int64_t>(h->sizes[l]) * h->sizes[l + 1] + h->sizes[l + 1];
    return n;
}

// Packed host layout: [W_0 {in,out} row-major, b_0 {1,out}, W_1, b_1, ...] without padding (what
// Module::named_parameters yields layer by layer, src/nn/models/mlp.cpp:32-33).
int odl_mlp_set_params(void *handle, const float *host_packed, void *stream)
{
    Mlp *h = H(handle);
    int64_t o = 0;
    for (int l = 0; l < h->L; ++l)
    {
        const int64_t nw = static_cast<int64_t>(h->sizes[l]) * h->sizes[l + 1], nb = h->sizes[l + 1];
        ODL_CUDA_TRY(cudaMemcpyAsync(h->params + h->w_off[l], host_packed + o, nw * 4, cudaMemcpyHostToDevice, ST(stream)));
        o += nw;
        ODL_CUDA_TRY(cudaMemcpyAsync(h->params + h->b_off[l], host_packed + o, nb * 4, cudaMemcpyHostToDevice, ST(stream)));
        o += nb;
    }
    if (three(h))
    {
        int rc = split_launch(h->params, h->total, 1, (int)h->total, nullptr, 0, nullptr, h->params_small, h->total,
                              nullptr, ST(stream));
        if (rc)
            return rc;
    }
    h->step_count = 0;
    ODL_CUDA_TRY(cudaMemsetAsync(h->m, 0, h->total * 4, ST(stream)));
    if (h->v)
        ODL_CUDA_TRY(cudaMemsetAsync(h->v, 0, h->total * 4, ST(stream)));
    ODL_CUDA_TRY(cudaStreamSynchronize(ST(stream)));
    return kOk;
}

// which: 0 parameters, 1 gradients of the last backward (after the optimizer's hook, like Parameter::grad()),
// 2 first-moment buffer (Adam m / SGD momentum buffer), 3 Adam's second moment.
int odl_mlp_get_packed(void *handle, int which, float *host_packed, void *stream)
{
    Mlp *h           = H(handle);
    const float *src = which == 0 ? h->params : which == 1 ? h->grads : which == 2 ? h->m : which == 3 ? h->v : nullptr;
    if (!src || !host_packed)
    {
        set_last_error("mlp_get_packed: buffer %d does not exist for this optimizer", which);
        return kInvalidArgument;
    }
    int64_t o = 0;
    for (int l = 0; l < h->L; ++l)
    {
        const int64_t nw = static_cast<int64_t>(h->sizes[l]) * h->sizes[l + 1], nb = h->sizes[l + 1];
        ODL_CUDA_TRY(cudaMemcpyAsync(host_packed + o, src + h->w_off[l], nw * 4, cudaMemcpyDeviceToHost, ST(stream)));
        o += nw;
        ODL_CUDA_TRY(cudaMemcpyAsync(host_packed + o, src + h->b_off[l], nb * 4, cudaMemcpyDeviceToHost, ST(stream)));
        o += nb;
    }
    ODL_CUDA_TRY(cudaStreamSynchronize(ST(stream)));
    return kOk;
}

// Restore the optimizer state saved with odl_mlp_get_packed(2 / 3) and odl_mlp_step_count: packed HOST arrays in the
// parameter order; v_packed is ignored (may be NULL) for SGD.  Call after odl_mlp_set_params, which zeroes the state.
int odl_mlp_set_optimizer_state(void *handle, const float *m_packed, const float *v_packed, int step_count, void *stream)
{
    Mlp *h = H(handle);
    if (!m_packed || step_count < 0 || (h->optimizer == 1 && !v_packed))
    {
        set_last_error("mlp_set_optimizer_state: invalid argument (step_count=%d)", step_count);
        return kInvalidArgument;
    }
    const float *srcs[2] = {m_packed, h->optimizer == 1 ? v_packed : nullptr};
    float *dsts[2]       = {h->m, h->v};
    for (int k = 0; k < 2; ++k)
    {
        if (!srcs[k] || !dsts[k])
            continue;
        int64_t o = 0;
        for (int l = 0; l < h->L; ++l)
        {
            const int64_t nw = static_cast<int64_t>(h->sizes[l]) * h->sizes[l + 1], nb = h->sizes[l + 1];
            ODL_CUDA_TRY(cudaMemcpyAsync(dsts[k] + h->w_off[l], srcs[k] + o, nw * 4, cudaMemcpyHostToDevice, ST(stream)));
            o += nw;
            ODL_CUDA_TRY(cudaMemcpyAsync(dsts[k] + h->b_off[l], srcs[k] + o, nb * 4, cudaMemcpyHostToDevice, ST(stream)));
            o += nb;
        }
    }
    h->step_count = step_count;
    ODL_CUDA_TRY(cudaStreamSynchronize(ST(stream)));
    return kOk;
}

// Optimizer steps taken since the parameters were installed (Adam's t).
int64_t odl_mlp_step_count(void *handle)
{
    return H(handle)->step_count;
}

// Forward through all layers, loss and d loss / d logits (scaled by grad_scale / batch), bias gradient of the head.
int odl_mlp_forward_loss(void *handle, const float *x, const void *labels, int labels_are_int64, void *stream)
{
    Mlp *h         = H(handle);
    cudaStream_t s = ST(stream);
    const int64_t B = h->batch;
    int rc;
    NvtxRange range("odl forward + loss");
    h->cur_x = x;
    if (three(h))
    {
        rc = split_launch(x, h->sizes[0], (int)B, h->sizes[0], nullptr, 0, nullptr, h->x_small, h->sizes[0], nullptr, s);
        if (rc)
            return rc;
    }
    const float *in = x, *in_s = h->x_small;
    for (int l = 0; l < h->L; ++l)
    {
        const bool last = (l + 1 == h->L);
        rc = linear_forward(in, in_s, h->params + h->w_off[l], three(h) ? h->params_small + h->w_off[l] : nullptr,
                            h->params + h->b_off[l], h->act[l], last ? nullptr : h->act_small[l], B, h->sizes[l + 1],
                            h->sizes[l], ODL_W_IN_OUT, last ? 0 : 1, h->precision, s);
        if (rc)
            return rc;
        in = h->act[l], in_s = h->act_small[l];
    }
    const int C = h->sizes[h->L];
    rc = softmax_ce_launch(h->act[h->L - 1], labels_are_int64 ? nullptr : static_cast<const int32_t *>(labels),
                           labels_are_int64 ? static_cast<const int64_t *>(labels) : nullptr, B, C, h->loss, h->gbuf[0],
                           h->row_loss, 1.0f, s);
    if (rc)
        return rc;
    // low part of dlogits + bias gradient of the head in one pass
    float *db = h->grads + h->b_off[h->L - 1];
    ODL_CUDA_TRY(cudaMemsetAsync(db, 0, static_cast<size_t>(C) * 4, s));
    return split_launch(h->gbuf[0], C, (int)B, C, nullptr, 0, nullptr, three(h) ? h->gbuf_small[0] : nullptr, C, db, s);
}

// Backward of layer `layer` (call for layer = L-1 ... 0): dW_layer into the flat gradient buffer and, for layer > 0,
// the gradient w.r.t. the layer below's pre-activation together with that layer's bias gradient.
}  // extern "C"

namespace odl
{
namespace
{
// Backward of one layer.  dw_done (optional): dW is computed before dX and the event recorded right behind its GEMM.
int backward_layer(Mlp *h, int layer, cudaStream_t s, cudaEvent_t dw_done)
{
    if (layer < 0 || layer >= h->L)
    {
        set_last_error("mlp: layer %d out of range", layer);
        return kInvalidArgument;
    }
    const int64_t B  = h->batch;
    NvtxRange range("odl backward layer", layer);
    const int cur    = (h->L - 1 - layer) & 1;  // ping-pong: the head's gradient sits in gbuf[0]
    const float *g   = h->gbuf[cur], *g_s = h->gbuf_small[cur];
    const float *xin = layer == 0 ? h->cur_x : h->act[layer - 1];
    const float *xin_s = layer == 0 ? h->x_small : h->act_small[layer - 1];
    float *dx = nullptr, *dx_s = nullptr, *prev_db = nullptr;
    const float *prev_y = nullptr;
    if (layer > 0)
    {
        dx      = h->gbuf[cur ^ 1];
        dx_s    = three(h) ? h->gbuf_small[cur ^ 1] : nullptr;
        prev_y  = h->act[layer - 1];
        prev_db = h->grads + h->b_off[layer - 1];
    }
    return linear_backward(xin, xin_s, h->params + h->w_off[layer], three(h) ? h->params_small + h->w_off[layer] : nullptr,
                           g, g_s, nullptr, dx, dx_s, prev_y, prev_db, h->grads + h->w_off[layer], nullptr, B,
                           h->sizes[layer + 1], h->sizes[layer], ODL_W_IN_OUT, h->precision, s, dw_done);
}

// The optimizer's update of the flat range [o, o + n) (any range: the update is elementwise).
int update_range(Mlp *h, int64_t o, int64_t n, float grad_scale, cudaStream_t s)
{
    float *ps = h->params_small ? h->params_small + o : nullptr;
    if (h->optimizer == 1)
        return adam_launch(h->params + o, h->grads + o, h->m + o, h->v + o, ps, n, h->step_count, h->lr, h->beta1, h->beta2,
                           h->eps, h->hook_wd, grad_scale, s);
    return sgd_launch(h->params + o, h->grads + o, h->m ? h->m + o : nullptr, ps, n, h->lr, h->momentum, 0.0f, 0, h->hook_wd,
                      grad_scale, s);
}
}  // namespace
}  // namespace odl

extern "C" {

int odl_mlp_backward_layer(void *handle, int layer, void *stream)
{
    return backward_layer(H(handle), layer, ST(stream), nullptr);
}

// One fused update of every parameter.  grad_scale: 1/world_size after a summing all-reduce, else 1.
int odl_mlp_optimizer_step(void *handle, float grad_scale, void *stream)
{
    Mlp *h = H(handle);
    NvtxRange range("odl optimizer");
    h->step_count += 1;
    if (h->optimizer == 1)
        return adam_launch(h->params, h->grads, h->m, h->v, h->params_small, h->total, h->step_count, h->lr, h->beta1,
                           h->beta2, h->eps, h->hook_wd, grad_scale, ST(stream));
    return sgd_launch(h->params, h->grads, h->m, h->params_small, h->total, h->lr, h->momentum, 0.0f, 0, h->hook_wd,
                      grad_scale, ST(stream));
}

// The same update restricted to the parameters of one layer ([W_layer, b_layer], contiguous in the flat buffers), so that a
// data-parallel caller can update every layer as soon as ITS gradient bucket has been reduced -- the updates of the
// layers reduced early then overlap the all-reduce of the last bucket.  Call once per layer and step, in any order;
// first_of_step != 0 on the first call of a step advances the step counter (Adam's t) that all layers of the step share.
int odl_mlp_optimizer_step_layer(void *handle, int layer, float grad_scale, int first_of_step, void *stream)
{
    Mlp *h = H(handle);
    if (layer < 0 || layer >= h->L)
    {
        set_last_error("mlp: layer %d out of range", layer);
        return kInvalidArgument;
    }
    if (first_of_step)
        h->step_count += 1;
    NvtxRange range("odl optimizer layer", layer);
    const int64_t o = h->w_off[layer];
    const int64_t n = (layer + 1 < h->L ? h->w_off[layer + 1] : h->total) - o;
    float *ps       = h->params_small ? h->params_small + o : nullptr;
    if (h->optimizer == 1)
        return adam_launch(h->params + o, h->grads + o, h->m + o, h->v + o, ps, n, h->step_count, h->lr, h->beta1, h->beta2,
                           h->eps, h->hook_wd, grad_scale, ST(stream));
    return sgd_launch(h->params + o, h->grads + o, h->m ? h->m + o : nullptr, ps, n, h->lr, h->momentum, 0.0f, 0, h->hook_wd,
                      grad_scale, ST(stream));
}

int odl_mlp_train_step(void *handle, const float *x, const void *labels, int labels_are_int64, void *stream)
{
    int rc = odl_mlp_forward_loss(handle, x, labels, labels_are_int64, stream);
    if (rc)
        return rc;
    for (int l = H(handle)->L - 1; l >= 0; --l)
        if ((rc = odl_mlp_backward_layer(handle, l, stream)))
            return rc;
    // One update of the whole buffer behind backward.  (Measured: running layer l's update on a second stream as soon as
    // its backward is done gains nothing -- 51.37 against 51.36 ms on the benchmark step: a persistent GEMM CTA holds nearly
    // all of its SM's shared memory and most of its registers, so the update mostly runs between two GEMMs either way.)
    return odl_mlp_optimizer_step(handle, 1.0f, stream);
}

// ---- data-parallel step -------------------------------------------------------------------------------------------
int odl_mlp_dp_attach(void *handle, void *comm, int dw0_panels)
{
    Mlp *h = H(handle);
    if (!h || !comm || dw0_panels < 0 || dw0_panels > 8)
    {
        set_last_error("mlp_dp_attach: invalid argument (dw0_panels=%d)", dw0_panels);
        return kInvalidArgument;
    }
    h->drop_dp();
    Comm *c = static_cast<Comm *>(comm);
    // Row panels of dW_0 {in, out}: rows [k0, k1) are a contiguous range of the flat gradient buffer and one GEMM on the
    // columns k0 ... k1 of x.  Worth it only where the bucket is large and other ranks exist; every panel must keep the
    // 32-column granularity of the one-copy-per-operand tensor maps.
    const int64_t in0 = h->sizes[0], out0 = h->sizes[1];
    int panels = dw0_panels;
    if (panels == 0)
        panels = (comm_world(c) > 1 && in0 * out0 >= (int64_t(1) << 24)) ? 4 : 1;
    while (panels > 1 && (in0 % (32 * panels) != 0))
        --panels;
    h->dw0_panels = panels;
    // The communication stream gets the highest priority: when a GEMM ends and both the next GEMM and a waiting
    // all-reduce could start, the all-reduce's few blocks are placed first and the GEMM takes the remaining SMs (its
    // pairs draw their tiles from a counter, so it does not wait for the ones that start late).
    int prio_least = 0, prio_greatest = 0;
    ODL_CUDA_TRY(cudaDeviceGetStreamPriorityRange(&prio_least, &prio_greatest));
    ODL_CUDA_TRY(cudaStreamCreateWithPriority(&h->comm_stream, cudaStreamNonBlocking, prio_greatest));
    const int pieces = (h->L - 1) + panels;
    for (int i = 0; i < pieces; ++i)
    {
        cudaEvent_t a = nullptr, b = nullptr;
        ODL_CUDA_TRY(cudaEventCreateWithFlags(&a, cudaEventDisableTiming));
        h->ev_ready.push_back(a);
        ODL_CUDA_TRY(cudaEventCreateWithFlags(&b, cudaEventDisableTiming));
        h->ev_reduced.push_back(b);
    }
    for (int l = 0; l < h->L; ++l)
    {
        cudaEvent_t e = nullptr;
        ODL_CUDA_TRY(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        h->ev_layer_done.push_back(e);
    }
    ODL_CUDA_TRY(cudaEventCreateWithFlags(&h->ev_step_done, cudaEventDisableTiming));
    h->comm = c;
    return kOk;
}

namespace
{
// Step timeline for tuning the overlap (environment variable ODL_DP_TRACE=1): timing events on both streams, printed to
// stderr after the step has drained -- the one synchronisation it adds sits after everything was enqueued.
struct DpTrace
{
    struct Mark
    {
        cudaEvent_t ev;
        char what[48];
    };
    std::vector<Mark> marks;
    bool on = false;
    void begin()
    {
        static const bool enabled = [] {
            const char *e = std::getenv("ODL_DP_TRACE");
            return e && *e && *e != '0';
        }();
        on = enabled;
        marks.clear();
    }
    void mark(cudaStream_t st, const char *what, int a)
    {
        if (!on)
            return;
        Mark m;
        if (cudaEventCreate(&m.ev) != cudaSuccess)
            return;
        std::snprintf(m.what, sizeof(m.what), "%s %d", what, a);
        cudaEventRecord(m.ev, st);
        marks.push_back(m);
    }
    void print(cudaStream_t a, cudaStream_t b, int rank)
    {
        if (!on || marks.empty())
            return;
        cudaStreamSynchronize(a);
        cudaStreamSynchronize(b);
        for (size_t i = 0; i < marks.size(); ++i)
        {
            float ms = 0.f;
            cudaEventElapsedTime(&ms, marks[0].ev, marks[i].ev);
            std::fprintf(stderr, "[odl dp trace, rank %d] %8.3f ms  %s\n", rank, ms, marks[i].what);
        }
        for (auto &m : marks)
            cudaEventDestroy(m.ev);
        marks.clear();
    }
};
thread_local DpTrace g_trace;

// Piece i's gradients are final on `s`: sum them over the ranks on the communication stream.
// (ev_ready[piece] has been recorded behind the GEMM that made them final.)
int reduce_piece(Mlp *h, int piece, float *ptr, int64_t count, int layer)
{
    NvtxRange range("odl all-reduce layer", layer);
    ODL_CUDA_TRY(cudaStreamWaitEvent(h->comm_stream, h->ev_ready[piece], 0));
    g_trace.mark(h->comm_stream, "  comm: all-reduce may start, piece", piece);
    int rc = comm_allreduce_sum(h->comm, ptr, count, h->comm_stream);
    if (rc)
        return rc;
    g_trace.mark(h->comm_stream, "  comm: all-reduce done, piece", piece);
    ODL_CUDA_TRY(cudaEventRecord(h->ev_reduced[piece], h->comm_stream));
    return kOk;
}
}  // namespace

int odl_mlp_train_step_dp(void *handle, const float *x, const void *labels, int labels_are_int64, void *stream)
{
    Mlp *h = H(handle);
    if (!h->comm)
    {
        set_last_error("mlp_train_step_dp: odl_mlp_dp_attach has not been called");
        return kInvalidArgument;
    }
    cudaStream_t s = ST(stream);
    g_trace.begin();
    g_trace.mark(s, "step start", 0);
    int rc = odl_mlp_forward_loss(handle, x, labels, labels_are_int64, stream);
    if (rc)
        return rc;
    g_trace.mark(s, "forward + loss done", 0);
    // Head first.  Bucket l = [dW_l, db_l] (db_l came out of layer l+1's dX epilogue) is final after layer l's dW GEMM,
    // which runs BEFORE its dX GEMM here: the all-reduce of bucket l starts behind dW_l and has dX_l and everything below to
    // hide behind.  The communication stream also runs the updates: layer l's as soon as its bucket is reduced and its dX
    // GEMM (the last reader of W_l) has finished.
    const float scale = 1.0f / static_cast<float>(comm_world(h->comm));
    h->step_count += 1;
    for (int l = h->L - 1; l >= 1; --l)
    {
        const int piece = h->L - 1 - l;
        if ((rc = backward_layer(h, l, s, h->ev_ready[piece])))
            return rc;
        g_trace.mark(s, "backward done, layer", l);
        const int64_t o = h->w_off[l];
        const int64_t n = (l + 1 < h->L ? h->w_off[l + 1] : h->total) - o;
        if ((rc = reduce_piece(h, piece, h->grads + o, n, l)))
            return rc;
        ODL_CUDA_TRY(cudaEventRecord(h->ev_layer_done[l], s));
        ODL_CUDA_TRY(cudaStreamWaitEvent(h->comm_stream, h->ev_layer_done[l], 0));
        if ((rc = update_range(h, o, n, scale, h->comm_stream)))
            return rc;
        g_trace.mark(h->comm_stream, "  comm: update done, layer", l);
    }
    // layer 0 has no dX: its backward is the one GEMM dW_0{in,out} = x^T . g, done here in dw0_panels row panels (rows
    // [k0, k1) are a contiguous range of the flat gradient buffer), each reduced and updated as soon as it is final
    const int first0 = h->L - 1;  // piece index of layer 0's first panel
    {
        const int64_t B = h->batch, in0 = h->sizes[0], out0 = h->sizes[1];
        const int cur   = (h->L - 1) & 1;
        const float *g = h->gbuf[cur], *g_s = three(h) ? h->gbuf_small[cur] : nullptr;
        const int64_t rows = in0 / h->dw0_panels;
        const int64_t end  = (h->L > 1 ? h->w_off[1] : h->total);  // the last panel carries db_0 and the padding
        for (int p = 0; p < h->dw0_panels; ++p)
        {
            NvtxRange range("odl backward layer 0 panel", p);
            const int64_t k0 = p * rows;
            rc = gemm_dispatch(1, 0, rows, out0, B, h->cur_x + k0, three(h) ? h->x_small + k0 : nullptr, in0, g, g_s, out0,
                               h->grads + h->w_off[0] + k0 * out0, nullptr, out0, nullptr, nullptr, 0, nullptr, 0,
                               h->precision, s, true);
            if (rc)
                return rc;
            g_trace.mark(s, "backward done, layer 0 panel", p);
            ODL_CUDA_TRY(cudaEventRecord(h->ev_ready[first0 + p], s));
            const int64_t lo = h->w_off[0] + k0 * out0;
            const int64_t hi = (p + 1 == h->dw0_panels) ? end : h->w_off[0] + (k0 + rows) * out0;
            if ((rc = reduce_piece(h, first0 + p, h->grads + lo, hi - lo, 0)))
                return rc;
            if ((rc = update_range(h, lo, hi - lo, scale, h->comm_stream)))
                return rc;
            g_trace.mark(h->comm_stream, "  comm: update done, layer 0 panel", p);
        }
    }
    // the step is complete when the communication stream is: odl_mlp_dp_wait watches this event
    ODL_CUDA_TRY(cudaEventRecord(h->ev_step_done, h->comm_stream));
    ODL_CUDA_TRY(cudaStreamWaitEvent(s, h->ev_step_done, 0));
    g_trace.print(s, h->comm_stream, comm_rank(h->comm));
    return kOk;
}

int odl_mlp_dp_wait(void *handle, int timeout_ms)
{
    Mlp *h = H(handle);
    if (!h->comm || h->ev_reduced.empty())
    {
        set_last_error("mlp_dp_wait: odl_mlp_dp_attach has not been called");
        return kInvalidArgument;
    }
    // the communication stream runs its collectives and updates in order: its last event covers the whole step
    cudaEvent_t last = h->ev_step_done;
    auto done = [](void *ev) -> int { return cudaEventQuery(static_cast<cudaEvent_t>(ev)) != cudaErrorNotReady ? 1 : 0; };
    return comm_watch(h->comm, timeout_ms, done, last);
}

// Whole-step CUDA graph: records forward + loss + backward of every layer on the given STATIC input buffers into one
// graph (the optimizer launch stays outside: Adam's bias corrections are host scalars that change every step).  One
// un-recorded forward + backward runs first so that every scratch buffer has its final size -- allocation cannot be
// captured; parameters and optimizer state are not touched by it.  `stream` must be a real (non-default) stream; the
// capture is thread-local, so other threads (a loader copying the next batch) are not disturbed.  The caller refills x
// and labels in place between odl_mlp_replay calls.
int odl_mlp_capture(void *handle, const float *x, const void *labels, int labels_are_int64, void *stream)
{
    Mlp *h = H(handle);
    if (!stream)
    {
        set_last_error("mlp capture: needs a non-default stream");
        return kInvalidArgument;
    }
    cudaStream_t s = ST(stream);
    auto record = [&]() -> int {
        int rc = odl_mlp_forward_loss(handle, x, labels, labels_are_int64, stream);
        for (int l = h->L - 1; l >= 0 && !rc; --l)
            rc = odl_mlp_backward_layer(handle, l, stream);
        return rc;
    };
    int rc = record();  // warm-up: sizes the scratch buffers, sets the kernels' attributes
    if (rc)
        return rc;
    ODL_CUDA_TRY(cudaStreamSynchronize(s));
    if (h->step_graph)
    {
        cudaGraphExecDestroy(h->step_graph);
        h->step_graph = nullptr;
    }
    const long long before     = g_launch_count;
    const long long generation = scratch_generation();
    ODL_CUDA_TRY(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
    rc = record();
    cudaGraph_t graph = nullptr;
    cudaError_t e     = cudaStreamEndCapture(s, &graph);
    h->graph_launches = g_launch_count - before;
    g_launch_count    = before;  // recorded, not run
    if (rc || e != cudaSuccess || !graph)
    {
        if (graph)
            cudaGraphDestroy(graph);
        if (!rc)
            set_last_error("mlp capture: cudaStreamEndCapture failed: %s", cudaGetErrorString(e));
        return rc ? rc : kCudaError;
    }
    e = cudaGraphInstantiate(&h->step_graph, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess)
    {
        h->step_graph = nullptr;
        set_last_error("mlp capture: cudaGraphInstantiate failed: %s", cudaGetErrorString(e));
        return kCudaError;
    }
    if (scratch_generation() != generation)
    {
        // cannot happen after the sizing pass above (growing drains the device, which a capture refuses); kept as a guard
        cudaGraphExecDestroy(h->step_graph);
        h->step_graph = nullptr;
        set_last_error("mlp capture: scratch memory was replaced while recording");
        return kStaleGraph;
    }
    h->graph_generation = generation;
    return kOk;
}

// One optimisation step from the recorded graph: replay, then the optimizer launch.
int odl_mlp_replay(void *handle, void *stream)
{
    Mlp *h = H(handle);
    if (!h->step_graph)
    {
        set_last_error("mlp replay: odl_mlp_capture has not been called");
        return kInvalidArgument;
    }
    if (scratch_generation() != h->graph_generation)
    {
        set_last_error("mlp replay: the library's scratch memory was replaced after odl_mlp_capture (a later call needed "
                       "more of it); the recorded step holds stale addresses -- call odl_mlp_capture again");
        return kStaleGraph;
    }
    ODL_CUDA_TRY(cudaGraphLaunch(h->step_graph, ST(stream)));
    g_launch_count += h->graph_launches;
    return odl_mlp_optimizer_step(handle, 1.0f, stream);
}

// Device pointer of the scalar loss of the last forward (read it after synchronising the stream).
float *odl_mlp_loss_ptr(void *handle)
{
    return H(handle)->loss;
}

// Logits of the last forward: device pointer to [batch, sizes.back()].
float *odl_mlp_logits_ptr(void *handle)
{
    Mlp *h = H(handle);
    return h->act[h->L - 1];
}

// Contiguous gradient range [dW_layer, db_layer] (device pointer, element count) for the data-parallel all-reduce;
// layer = -1 gives the whole flat gradient buffer.
int odl_mlp_grad_bucket(void *handle, int layer, float **ptr, int64_t *count)
{
    Mlp *h = H(handle);
    if (layer < -1 || layer >= h->L || !ptr || !count)
    {
        set_last_error("mlp: bad bucket request");
        return kInvalidArgument;
    }
    if (layer == -1)
    {
        *ptr   = h->grads;
        *count = h->total;
        return kOk;
    }
    *ptr   = h->grads + h->w_off[layer];
    *count = (layer + 1 < h->L ? h->w_off[layer + 1] : h->total) - h->w_off[layer];
    return kOk;
}

// Test hook: NVTX ranges opened so far in this process (0 unless ODL_NVTX is set).
long long odl_debug_nvtx_ranges(void)
{
    return nvtx_range_count();
}

}  // extern "C"
