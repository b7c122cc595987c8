// TEST INFRASTRUCTURE, not product code.
//
// Thin extern "C" driver around the UNMODIFIED OriginDL reference library (its
// CPU backend), so that Python tests and the CPU-baseline leg of the benchmark
// can push seeded host buffers through the reference's own public API
// (origin::Tensor, functional::*, nn::MLP, optim::Adam/SGD) and read fp32
// results back.  Nothing here restates any arithmetic: every number comes out
// of the reference's operators.  Built by oracle/Makefile into
// oracle/_ref/libodl_ref.so from the reference sources where they lie.
//
// Reference entry points used:
//   functional::mat_mul            src/operators/math/mat_mul.cpp:12-182
//   functional::transpose          src/operators/shape/transpose.cpp
//   functional::broadcast_to       src/operators/math/broadcast_to.cpp:10-46
//   functional::relu               src/operators/activation/relu.cpp:13-54
//   functional::softmax_cross_entropy  src/operators/loss/softmax_cross_entropy.cpp:17-111
//   functional::conv2d             src/operators/conv/conv2d.cpp:14-89
//   functional::custom_linear      src/operators/custom/linear.cpp:123-144
//   nn::MLP                        src/nn/models/mlp.cpp:11-61
//   Adam / SGD / WeightDecay       src/optim/adam.cpp, src/optim/sgd.cpp, include/origin/optim/hooks.h
//   save / load / load_checkpoint  src/io/model_io.cpp:114-273, src/io/checkpoint.cpp:15-226
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#include "origin/core/operator.h"
#include "origin/core/parameter.h"
#include "origin/core/tensor.h"
#include "origin/io/checkpoint.h"
#include "origin/io/model_io.h"
#include "origin/nn/layers/batch_norm2d.h"
#include "origin/nn/models/mlp.h"
#include "origin/optim/adam.h"
#include "origin/optim/hooks.h"
#include "origin/optim/sgd.h"

using namespace origin;
namespace F = origin::functional;

namespace
{
thread_local std::string g_err;

Tensor make(const float *p, std::initializer_list<size_t> dims, bool grad)
{
    Shape s(dims);
    std::vector<float> v(p, p + s.elements());
    return Tensor(v, s, dtype(DataType::kFloat32).requires_grad(grad));
}

void dump(const Tensor &t, float *out)
{
    if (!out)
        return;
    auto v = t.to_vector<float>();
    std::memcpy(out, v.data(), v.size() * sizeof(float));
}

template <typename Fn>
int guarded(Fn &&fn)
{
    try
    {
        fn();
        return 0;
    }
    catch (const std::exception &e)
    {
        g_err = e.what();
        return 1;
    }
    catch (...)
    {
        g_err = "unknown exception";
        return 2;
    }
}
}  // namespace

extern "C" {

const char *odlref_last_error()
{
    return g_err.c_str();
}

// C[M,N] = A[M,K] . B[K,N]  (row-major), through functional::mat_mul.
int odlref_matmul(const float *a, const float *b, float *c, int64_t M, int64_t N, int64_t K)
{
    return guarded([&] {
        auto A = make(a, {(size_t)M, (size_t)K}, false);
        auto B = make(b, {(size_t)K, (size_t)N}, false);
        dump(F::mat_mul(A, B), c);
    });
}

// MatMul backward with upstream gradient gy: gA = gy.B^T, gB = A^T.gy.
int odlref_matmul_backward(const float *a, const float *b, const float *gy, float *ga, float *gb, int64_t M,
                           int64_t N, int64_t K)
{
    return guarded([&] {
        auto A  = make(a, {(size_t)M, (size_t)K}, true);
        auto B  = make(b, {(size_t)K, (size_t)N}, true);
        auto GY = make(gy, {(size_t)M, (size_t)N}, false);
        auto L  = F::sum(F::mat_mul(A, B) * GY);
        L.backward();
        dump(A.grad(), ga);
        dump(B.grad(), gb);
    });
}

// Forward-only fused Linear of the reference: y = x.W^T + b, W is [N,K], b is [N] (may be null).
int odlref_custom_linear(const float *x, const float *w, const float *b, float *y, int64_t M, int64_t N, int64_t K)
{
    return guarded([&] {
        auto X = make(x, {(size_t)M, (size_t)K}, false);
        auto W = make(w, {(size_t)N, (size_t)K}, false);
        if (b)
        {
            auto Bv = make(b, {(size_t)N}, false);
            dump(F::custom_linear(X, W, Bv, (int)K, (int)N, true), y);
        }
        else
        {
            dump(F::custom_linear(X, W, (int)K, (int)N), y);
        }
    });
}

// Linear forward + backward composed from the reference's autograd operators.
// w_layout 0: W is [N,K]  (y = x.transpose(W) + b) ; 1: W is [K,N] as nn::Linear stores it (y = x.W + b).
// relu != 0 applies functional::relu to the result.  dY is injected as loss = sum(y * dY).
int odlref_linear_fwd_bwd(const float *x, const float *w, const float *b, const float *dy, int64_t M, int64_t N,
                          int64_t K, int w_layout, int relu, float *y, float *dx, float *dw, float *db)
{
    return guarded([&] {
        auto X = make(x, {(size_t)M, (size_t)K}, true);
        auto W = w_layout == 0 ? make(w, {(size_t)N, (size_t)K}, true) : make(w, {(size_t)K, (size_t)N}, true);
        Tensor Bv;
        if (b)
            Bv = make(b, {1, (size_t)N}, true);
        Tensor out = w_layout == 0 ? F::mat_mul(X, F::transpose(W)) : F::mat_mul(X, W);
        if (b)
            out = out + F::broadcast_to(Bv, out.shape());
        if (relu)
            out = F::relu(out);
        dump(out, y);
        if (dy)
        {
            auto DY = make(dy, {(size_t)M, (size_t)N}, false);
            auto L  = F::sum(out * DY);
            L.backward();
            dump(X.grad(), dx);
            dump(W.grad(), dw);
            if (b)
                dump(Bv.grad(), db);
        }
    });
}

// loss = softmax_cross_entropy(logits[B,C], labels[B]); dlogits = d loss / d logits.
int odlref_softmax_ce(const float *logits, const int32_t *labels, int64_t B, int64_t C, float *loss, float *dlogits)
{
    return guarded([&] {
        auto X = make(logits, {(size_t)B, (size_t)C}, true);
        std::vector<int32_t> tv(labels, labels + B);
        Tensor T(tv, Shape{(size_t)B}, dtype(DataType::kInt32));
        auto L = F::softmax_cross_entropy(X, T);
        if (loss)
            *loss = L.item<float>();
        if (dlogits)
        {
            L.backward();
            dump(X.grad(), dlogits);
        }
    });
}

// conv2d forward + backward through functional::conv2d.  dY injected as sum(y*dY).
int odlref_conv2d_fwd_bwd(const float *x, const float *w, const float *b, const float *dy, int64_t N, int64_t C,
                          int64_t H, int64_t W_, int64_t OC, int64_t KH, int64_t KW, int stride, int pad, float *y,
                          float *dx, float *dw, float *db)
{
    return guarded([&] {
        auto X  = make(x, {(size_t)N, (size_t)C, (size_t)H, (size_t)W_}, true);
        auto Wt = make(w, {(size_t)OC, (size_t)C, (size_t)KH, (size_t)KW}, true);
        Tensor Bv;
        if (b)
            Bv = make(b, {(size_t)OC}, true);
        auto out = F::conv2d(X, Wt, b ? &Bv : nullptr, stride, pad);
        dump(out, y);
        if (dy)
        {
            std::vector<float> dv(dy, dy + out.elements());
            Tensor DY(dv, out.shape(), dtype(DataType::kFloat32));
            auto L = F::sum(out * DY);
            L.backward();
            dump(X.grad(), dx);
            dump(Wt.grad(), dw);
            if (b)
                dump(Bv.grad(), db);
        }
    });
}

// MLP training through nn::MLP + the reference optimizers.
//   sizes[n_sizes]      layer widths, e.g. {784,1000,1000,10}
//   params              concatenated per layer: W_i {in,out} row-major then b_i {1,out}; updated in place on return
//   x[steps_data][B,in], labels[steps_data][B]: batch s uses slot (s % n_batches)
//   opt: 0 = SGD(lr, momentum, weight_decay=0, nesterov=false), 1 = Adam(lr, .9, .999, 1e-8)
//   hook_wd > 0 registers the WeightDecay hook with that rate.
//   losses[steps] receives the loss of every step (value before the update).
//   grads (optional): gradients of the LAST step, same packing as params (after hooks ran).
int odlref_mlp_train(const int32_t *sizes, int n_sizes, float *params, const float *x, const int32_t *labels,
                     int64_t B, int n_batches, int steps, int opt, float lr, float momentum, float hook_wd,
                     float *losses, float *grads)
{
    return guarded([&] {
        std::vector<int> hs(sizes, sizes + n_sizes);
        nn::MLP model(hs);
        auto named = model.named_parameters("");
        size_t off = 0;
        std::vector<Parameter *> order;
        for (int i = 0; i + 1 < n_sizes; ++i)
        {
            size_t in = hs[i], out = hs[i + 1];
            auto *pw = named.at("layer_" + std::to_string(i) + ".weight");
            auto *pb = named.at("layer_" + std::to_string(i) + ".bias");
            *pw      = Parameter(make(params + off, {in, out}, true));
            off += in * out;
            *pb = Parameter(make(params + off, {1, out}, true));
            off += out;
            order.push_back(pw);
            order.push_back(pb);
        }
        std::unique_ptr<Optimizer> optim;
        if (opt == 0)
            optim = std::make_unique<SGD>(model, lr, momentum, 0.0f, false);
        else
            optim = std::make_unique<Adam>(model, lr);
        WeightDecay wd(hook_wd);
        if (hook_wd > 0.0f)
            optim->register_hook(wd.hook());

        size_t in0 = hs[0];
        for (int s = 0; s < steps; ++s)
        {
            int slot = s % n_batches;
            auto X   = make(x + (size_t)slot * B * in0, {(size_t)B, in0}, false);
            std::vector<int32_t> tv(labels + (size_t)slot * B, labels + (size_t)(slot + 1) * B);
            Tensor T(tv, Shape{(size_t)B}, dtype(DataType::kInt32));
            auto yv   = model(X);
            auto loss = F::softmax_cross_entropy(yv, T);
            losses[s] = loss.item<float>();
            optim->zero_grad();
            loss.backward();
            if (grads && s == steps - 1)
            {
                // hooks mutate grads inside step(); capture the raw backward result here
                size_t g = 0;
                for (auto *p : order)
                {
                    dump(p->grad(), grads + g);
                    g += p->elements();
                }
            }
            optim->step();
        }
        off = 0;
        for (auto *p : order)
        {
            dump(*p, params + off);
            off += p->elements();
        }
    });
}

// One optimizer step on a single parameter tensor of n elements with a given gradient.
// state: opt 0 (SGD) -> buf[n]; opt 1 (Adam) -> not exposed by the reference, so `steps` updates are replayed
// from zero state with the same gradient sequence grads[steps][n].  p is updated in place.
int odlref_optim_replay(float *p, const float *grads, int64_t n, int steps, int opt, float lr, float momentum,
                        float sgd_wd, int nesterov, float hook_wd)
{
    return guarded([&] {
        // A 1-layer bias-free module would add a matmul; drive the optimizer on a Linear's weight directly.
        nn::Linear lin(1, (int)n, false);
        *lin.weight() = Parameter(make(p, {1, (size_t)n}, true));
        std::unique_ptr<Optimizer> optim;
        if (opt == 0)
            optim = std::make_unique<SGD>(lin, lr, momentum, sgd_wd, nesterov != 0);
        else
            optim = std::make_unique<Adam>(lin, lr);
        WeightDecay wd(hook_wd);
        if (hook_wd > 0.0f)
            optim->register_hook(wd.hook());
        for (int s = 0; s < steps; ++s)
        {
            optim->zero_grad();
            // y = x.W with x = [[1]] gives dL/dW = gy; inject gy = grads[s].
            auto X  = Tensor(std::vector<float>{1.0f}, Shape{1, 1}, dtype(DataType::kFloat32));
            auto Y  = lin.forward(X);
            auto GY = make(grads + (size_t)s * n, {1, (size_t)n}, false);
            auto L  = F::sum(Y * GY);
            L.backward();
            optim->step();
        }
        dump(*lin.weight(), p);
    });
}

// ---- BatchNorm (+ ReLU / SiLU) through functional::BatchNorm, functional::relu / silu and nn::BatchNorm2d
//      (src/operators/normalization/batch_norm.cpp:18-140, src/operators/activation/silu.cpp, src/nn/layers/batch_norm2d.cpp)

// x is {N,C} when HW == 1 and {N,C,H,W} with H*W = HW otherwise (H = HW, W = 1 is used: the arithmetic only depends
// on H*W).  act: 0 none, 1 relu, 2 silu.  dy != NULL runs backward of sum(out * dy).  mean / var receive the batch
// statistics the operator returns in training mode.  x, gamma and beta always require grad: without that the operator
// takes its inference path and reports zeros as the batch statistics (batch_norm.cpp:55-63).
int odlref_batch_norm_fwd_bwd(const float *x, const float *gamma, const float *beta, const float *running_mean,
                              const float *running_var, int training, float eps, int64_t N, int64_t C, int64_t HW,
                              int act, const float *dy, float *y, float *mean, float *var, float *gx, float *dgamma,
                              float *dbeta)
{
    return guarded([&] {
        const bool four = HW > 1;
        Shape xs        = four ? Shape{(size_t)N, (size_t)C, (size_t)HW, 1} : Shape{(size_t)N, (size_t)C};
        std::vector<float> xv(x, x + N * C * HW);
        Tensor X(xv, xs, dtype(DataType::kFloat32).requires_grad(true));
        auto G  = make(gamma, {(size_t)C}, true);
        auto B  = make(beta, {(size_t)C}, true);
        auto RM = make(running_mean, {(size_t)C}, false);
        auto RV = make(running_var, {(size_t)C}, false);
        auto op = std::make_shared<F::BatchNorm>(training != 0, eps, 0.1f, four ? 4 : 2);
        auto outs = (*op)({X, G, B, RM, RV});
        Tensor out = outs[0];
        if (training && outs.size() >= 3)
        {
            dump(outs[1], mean);
            dump(outs[2], var);
        }
        if (act == 1)
            out = F::relu(out);
        else if (act == 2)
            out = F::silu(out);
        dump(out, y);
        if (dy)
        {
            std::vector<float> dv(dy, dy + N * C * HW);
            Tensor DY(dv, xs, dtype(DataType::kFloat32));
            auto L = F::sum(out * DY);
            L.backward();
            dump(X.grad(), gx);
            dump(G.grad(), dgamma);
            dump(B.grad(), dbeta);
        }
    });
}

// nn::BatchNorm2d: `steps` training-mode forwards over xs[steps][N,C,H*W] (updating the running statistics), then one
// evaluation-mode forward of probe[N,C,H*W] -> y.
int odlref_batch_norm2d_layer(const float *xs, int steps, const float *probe, int64_t N, int64_t C, int64_t HW, float eps,
                              float momentum, float *y)
{
    return guarded([&] {
        nn::BatchNorm2d bn((int)C, eps, momentum);
        Shape s{(size_t)N, (size_t)C, (size_t)HW, 1};
        bn.train();
        for (int k = 0; k < steps; ++k)
        {
            std::vector<float> v(xs + (size_t)k * N * C * HW, xs + (size_t)(k + 1) * N * C * HW);
            bn.forward(Tensor(v, s, dtype(DataType::kFloat32)));
        }
        bn.eval();
        std::vector<float> pv(probe, probe + N * C * HW);
        dump(bn.forward(Tensor(pv, s, dtype(DataType::kFloat32))), y);
    });
}

int odlref_silu_fwd_bwd(const float *x, const float *dy, int64_t n, float *y, float *gx)
{
    return guarded([&] {
        auto X   = make(x, {(size_t)n}, dy != nullptr);
        auto out = F::silu(X);
        dump(out, y);
        if (dy)
        {
            auto L = F::sum(out * make(dy, {(size_t)n}, false));
            L.backward();
            dump(X.grad(), gx);
        }
    });
}

// ---- .odl state-dict files and .ckpt checkpoint directories through the reference's own origin::save / origin::load
//      (src/io/model_io.cpp:114-273, src/io/checkpoint.cpp:15-226).

// Write n float32 tensors (names[i], rank ranks[i], dims flattened in `dims`, values data[i]) with origin::save.
int odlref_save_state(const char *path, int n, const char **names, const int *ranks, const int64_t *dims,
                      const float **data)
{
    return guarded([&] {
        StateDict sd;
        size_t d = 0;
        for (int i = 0; i < n; ++i)
        {
            std::vector<size_t> shp(dims + d, dims + d + ranks[i]);
            d += ranks[i];
            Shape s(shp);
            std::vector<float> v(data[i], data[i] + s.elements());
            sd[names[i]] = Tensor(v, s, dtype(DataType::kFloat32));
        }
        save(sd, path);
    });
}

// Names in a file read by origin::load, '\n'-separated, into buf (truncated to cap - 1 characters); *count = tensors.
int odlref_load_state_names(const char *path, char *buf, int64_t cap, int *count)
{
    return guarded([&] {
        StateDict sd = load(path);
        std::string all;
        for (auto &kv : sd)
            all += kv.first + "\n";
        *count = (int)sd.size();
        std::snprintf(buf, (size_t)cap, "%s", all.c_str());
    });
}

// One float32 tensor of a file read by origin::load: rank and dims (up to 8) always; values when out != NULL.
int odlref_load_state_tensor(const char *path, const char *name, int *rank, int64_t *dims, float *out)
{
    return guarded([&] {
        StateDict sd = load(path);
        auto it      = sd.find(name);
        if (it == sd.end())
            throw std::runtime_error(std::string("no tensor named ") + name);
        const Shape &s = it->second.shape();
        *rank          = (int)s.size();
        for (size_t i = 0; i < s.size() && i < 8; ++i)
            dims[i] = (int64_t)s[i];
        dump(it->second, out);
    });
}

// origin::save(Checkpoint) of an MLP's state dict built from packed parameters (model.odl + metadata.json).
int odlref_save_checkpoint(const char *path, const int *sizes, int n_sizes, const float *params, int epoch, int step,
                           float loss, const char *optimizer_type, float lr, float beta1, float beta2, float eps)
{
    return guarded([&] {
        std::vector<int> sz(sizes, sizes + n_sizes);
        nn::MLP model(sz);
        size_t off = 0;
        for (int l = 0; l + 1 < n_sizes; ++l)
        {
            auto named = model.named_parameters("");
            auto *w    = named.at("layer_" + std::to_string(l) + ".weight");
            auto *b    = named.at("layer_" + std::to_string(l) + ".bias");
            *w         = Parameter(make(params + off, {(size_t)sizes[l], (size_t)sizes[l + 1]}, true));
            off += w->elements();
            *b = Parameter(make(params + off, {1, (size_t)sizes[l + 1]}, true));
            off += b->elements();
        }
        Checkpoint ck;
        ck.model_state_dict          = model.state_dict();
        ck.epoch                     = epoch;
        ck.step                      = step;
        ck.loss                      = loss;
        ck.optimizer_type            = optimizer_type;
        ck.optimizer_config["lr"]    = lr;
        ck.optimizer_config["beta1"] = beta1;
        ck.optimizer_config["beta2"] = beta2;
        ck.optimizer_config["eps"]   = eps;
        save(ck, path);
    });
}

// origin::load_checkpoint: metadata fields and the number of tensors in the model state dict.
int odlref_load_checkpoint_meta(const char *path, int *epoch, int *step, float *loss, char *optimizer_type, int64_t cap,
                                float *cfg4, int *n_tensors)
{
    return guarded([&] {
        Checkpoint ck = load_checkpoint(path);
        *epoch        = ck.epoch;
        *step         = ck.step;
        *loss         = ck.loss;
        std::snprintf(optimizer_type, (size_t)cap, "%s", ck.optimizer_type.c_str());
        const char *keys[4] = {"lr", "beta1", "beta2", "eps"};
        for (int i = 0; i < 4; ++i)
            cfg4[i] = ck.optimizer_config.count(keys[i]) ? ck.optimizer_config.at(keys[i]) : -1.0f;
        *n_tensors = (int)ck.model_state_dict.size();
    });
}

}  // extern "C"
