// GPU test program for the C++ host layer (origindl_b200/host/origin.hpp).  The cases follow the reference's own
// unit tests for this path -- same inputs, same expected values, same tolerances -- so that they read like
// tests/unit_test/operator/test_{matmul,linear,relu,softmax_cross_entropy,conv2d,conv2d_transpose_output}.cpp,
// tests/unit_test/optim/test_{adam,weight_decay}.cpp and tests/unit_test/autograd/test_linear_regression.cpp of the
// reference, plus the cases the reference cannot run (LinearOp backward, fused MLP training, the memory pool).
#include <unistd.h>

#include <cmath>
#include <cstdio>
#include <functional>
#include <string>
#include <vector>

#include "origin.hpp"

using namespace origin;
namespace F = origin::functional;

static int g_failed = 0, g_checks = 0;
static const float kDefault = 1e-3f;  // TestTolerance::kDefault of the reference (tests/unit_test/common/test_utils.h)

#define EXPECT_TRUE(c)                                                          \
    do                                                                          \
    {                                                                           \
        ++g_checks;                                                             \
        if (!(c))                                                               \
        {                                                                       \
            ++g_failed;                                                         \
            std::printf("    FAILED %s:%d  %s\n", __FILE__, __LINE__, #c);      \
        }                                                                       \
    } while (0)
#define EXPECT_NEAR(a, b, tol) EXPECT_TRUE(std::fabs((a) - (b)) <= (tol))
#define EXPECT_THROW(stmt)                      \
    do                                          \
    {                                           \
        bool thrown = false;                    \
        try                                     \
        {                                       \
            stmt;                               \
        }                                       \
        catch (const std::exception &)          \
        {                                       \
            thrown = true;                      \
        }                                       \
        EXPECT_TRUE(thrown);                    \
    } while (0)

static void expect_tensor(const Tensor &t, const std::vector<float> &want, float tol = kDefault)
{
    auto v = t.to_vector<float>();
    EXPECT_TRUE(v.size() == want.size());
    for (size_t i = 0; i < v.size() && i < want.size(); ++i)
        EXPECT_NEAR(v[i], want[i], tol);
}

static Tensor T(std::vector<float> v, Shape s, bool grad = false)
{
    return Tensor(v, s, dtype(DataType::kFloat32).requires_grad(grad));
}

// ---- test_matmul.cpp
static void matmul_forward()
{
    expect_tensor(F::mat_mul(T({1, 2, 3, 4}, {2, 2}), T({5, 6, 7, 8}, {2, 2})), {19, 22, 43, 50});
    EXPECT_NEAR(F::mat_mul(T({1, 2}, {1, 2}), T({3, 4}, {2, 1})).item<float>(), 11.0f, kDefault);
    expect_tensor(F::mat_mul(T({1, 2, 3, 4, 5, 6}, {2, 3}), T({7, 8, 9, 10, 11, 12}, {3, 2})), {58, 64, 139, 154});
    EXPECT_THROW(F::mat_mul(T({1, 2, 3, 4}, {2, 2}), T({1, 2, 3}, {3, 1})));  // dimension mismatch throws
    // all-ones sweep incl. sizes that are no multiple of any tile (the reference's CUDA-only sweep)
    for (size_t n : {16u, 31u, 127u, 512u})
    {
        auto y = F::mat_mul(Tensor::ones(Shape{n, n}), Tensor::ones(Shape{n, n})).to_vector<float>();
        bool ok = true;
        for (float v : y)
            ok = ok && std::fabs(v - (float)n) <= kDefault;
        EXPECT_TRUE(ok);
    }
    expect_tensor(F::mat_mul(Tensor::ones(Shape{1, 1000}), Tensor::ones(Shape{1000, 1})), {1000.0f});
}
static void matmul_backward()
{
    auto x = T({1, 2, 3, 4}, {2, 2}, true), w = T({5, 6, 7, 8}, {2, 2}, true);
    auto y = F::mat_mul(x, w);
    y.backward();
    expect_tensor(x.grad(), {11, 15, 11, 15});
    expect_tensor(w.grad(), {4, 4, 6, 6});
}
// ---- test_linear.cpp (+ the backward the reference does not have)
static void linear_forward()
{
    auto y = F::custom_linear(T({1, 2, 3, 4, 5, 6}, {2, 3}), T({1, 0, 0, 0, 1, 0, 0, 0, 1, 1, 1, 1}, {4, 3}),
                              T({0, 0, 0, 0}, {4}), 3, 4, true);
    EXPECT_TRUE(y.shape() == (Shape{2, 4}));
    expect_tensor(y, {1, 2, 3, 6, 4, 5, 6, 15});
    expect_tensor(F::custom_linear(T({1, 2}, {1, 2}), T({1, 0, 0, 1}, {2, 2}), T({1, 2}, {2}), 2, 2, true), {2, 4});
    expect_tensor(F::custom_linear(T({1, 2}, {1, 2}), T({1, 0, 0, 1}, {2, 2}), 2, 2), {1, 2});
    EXPECT_THROW(F::custom_linear(T({1, 2, 3}, {1, 3}), T({1, 0, 0, 1}, {2, 2}), 2, 2));  // feature mismatch
}
static void linear_backward()
{
    // y = x.W^T + b, L = sum(y): dx = colsum(W) per row, dW = rows of colsum(x), db = M
    auto x = T({1, 2, 3, 4, 5, 6}, {2, 3}, true), w = T({1, 0, 0, 0, 1, 0, 0, 0, 1, 1, 1, 1}, {4, 3}, true);
    auto b = T({0, 0, 0, 0}, {4}, true);
    auto y = F::custom_linear(x, w, b, 3, 4, true);
    y.backward();
    expect_tensor(x.grad(), {2, 2, 2, 2, 2, 2});
    expect_tensor(w.grad(), {5, 7, 9, 5, 7, 9, 5, 7, 9, 5, 7, 9});
    expect_tensor(b.grad(), {2, 2, 2, 2});
}
// ---- test_relu.cpp
static void relu_cases()
{
    expect_tensor(F::relu(T({-1, 0, 1, 2}, {4})), {0, 0, 1, 2});
    expect_tensor(F::relu(T({1, 2, 3}, {3})), {1, 2, 3});
    auto x = T({-1, 0, 1, 2}, {4}, true);
    auto y = F::relu(x);
    y.backward();
    expect_tensor(x.grad(), {0, 0, 1, 1});  // relu'(0) = 0
}
// ---- test_softmax_cross_entropy.cpp
static void softmax_ce_cases()
{
    auto x = T({1, 1, 1}, {1, 3});
    Tensor t(std::vector<int32_t>{1}, Shape{1}, dtype(DataType::kInt32));
    EXPECT_NEAR(F::softmax_cross_entropy(x, t).item<float>(), std::log(3.0f), 0.01f);
    // gradient = (p - onehot) / N
    auto z = T({1, 2, 3, 1, 2, 3}, {2, 3}, true);
    Tensor t2(std::vector<int32_t>{0, 2}, Shape{2}, dtype(DataType::kInt32));
    auto loss = F::softmax_cross_entropy(z, t2);
    loss.backward();
    const float e1 = std::exp(1.f), e2 = std::exp(2.f), e3 = std::exp(3.f), s = e1 + e2 + e3;
    expect_tensor(z.grad(), {(e1 / s - 1) / 2, e2 / s / 2, e3 / s / 2, e1 / s / 2, e2 / s / 2, (e3 / s - 1) / 2}, 0.01f);
    Tensor bad(std::vector<int32_t>{5, 0}, Shape{2}, dtype(DataType::kInt32));
    EXPECT_THROW(F::softmax_cross_entropy(z, bad));             // out-of-range index throws
    Tensor t64(std::vector<int64_t>{0, 2}, Shape{2}, dtype(DataType::kInt64));
    EXPECT_NEAR(F::softmax_cross_entropy(z, t64).item<float>(), loss.item<float>(), 1e-6f);
    EXPECT_THROW(F::softmax_cross_entropy(T({1, 2, 3}, {3}), t));  // x must be 2-D
}
// ---- test_conv2d.cpp, test_conv2d_transpose_output.cpp
static void conv2d_cases()
{
    auto x = T({1, 2, 3, 4, 5, 6, 7, 8, 9}, {1, 1, 3, 3});
    expect_tensor(F::conv2d(x, T({1, 1, 1, 1}, {1, 1, 2, 2})), {12, 16, 24, 28});
    auto b = T({1}, {1});
    expect_tensor(F::conv2d(T({1, 2, 3, 4}, {1, 1, 2, 2}), T({1, 1, 1, 1}, {1, 1, 2, 2}), &b), {11});
    auto y2 = F::conv2d(x, T({1, 1, 1, 1, 2, 2, 2, 2}, {2, 1, 2, 2}));
    EXPECT_TRUE(y2.shape() == (Shape{1, 2, 2, 2}));
    expect_tensor(y2, {12, 16, 24, 28, 24, 32, 48, 56});
    // backward with gy = ones (as the reference's backward tests do): gW = sums of the input windows, gx = coverage
    auto xg = T({1, 2, 3, 4, 5, 6, 7, 8, 9}, {1, 1, 3, 3}, true);
    auto wg = T({1, 1, 1, 1}, {1, 1, 2, 2}, true);
    auto yg = F::conv2d(xg, wg);
    yg.backward();
    expect_tensor(wg.grad(), {12, 16, 24, 28});
    expect_tensor(xg.grad(), {1, 2, 1, 2, 4, 2, 1, 2, 1});
    EXPECT_THROW(F::conv2d(T({1, 2, 3, 4}, {1, 1, 2, 2}), T({1, 1, 1, 1, 1, 1, 1, 1, 1}, {1, 1, 3, 3})));  // OH <= 0
    EXPECT_THROW(F::conv2d(x, T({1, 1, 1, 1, 1, 1, 1, 1}, {1, 2, 2, 2})));                                 // channels
}
// ---- test_weight_decay.cpp, test_adam.cpp
static void weight_decay_and_adam()
{
    nn::Linear lin(1, 1, false);
    *lin.weight() = Parameter(T({1.0f}, {1, 1}, true));
    SGD sgd(lin, 0.01f, 0.0f, 0.0f, false);
    WeightDecay wd(0.1f);
    auto x = T({1.0f}, {1, 1}), target = T({2.0f}, {1, 1});
    auto y = lin(x);
    auto loss = (y - target) * (y - target);
    loss.backward();
    const float before = lin.weight()->grad().item<float>();
    EXPECT_NEAR(before, -2.0f, 1e-5f);
    std::vector<Parameter *> ps = {lin.weight()};
    wd.hook()(ps);
    EXPECT_NEAR(lin.weight()->grad().item<float>(), before + 0.1f * 1.0f, 1e-5f);

    nn::Linear lin2(1, 1, true);
    *lin2.weight() = Parameter(T({1.0f}, {1, 1}, true));
    Adam adam(lin2, 0.01f, 0.9f, 0.999f, 1e-8f);
    float prev = 1.0f;
    for (int s = 0; s < 3; ++s)  // MultipleSteps: the parameter keeps moving towards the target
    {
        adam.zero_grad();
        auto yy = lin2(x);
        auto l2 = (yy - target) * (yy - target);
        l2.backward();
        adam.step();
        const float w = lin2.weight()->item<float>();
        EXPECT_TRUE(w > prev);
        prev = w;
    }
    EXPECT_NEAR(prev, 1.0f + 3 * 0.01f, 2e-3f);  // the first Adam steps move by ~lr each
}
// ---- autograd/test_linear_regression.cpp: 200 GD steps reach w = 2, b = 5 within 0.1
static void linear_regression()
{
    const size_t n = 100;
    std::vector<float> xs(n), ys(n);
    std::mt19937 gen(0);
    std::uniform_real_distribution<float> u(0.f, 1.f);
    std::normal_distribution<float> noise(0.f, 0.05f);
    for (size_t i = 0; i < n; ++i)
    {
        xs[i] = u(gen);
        ys[i] = 2.0f * xs[i] + 5.0f + noise(gen);
    }
    auto x = T(xs, {n, 1}), y = T(ys, {n, 1});
    auto w = T({0.0f}, {1, 1}, true), b = T({0.0f}, {1, 1}, true);
    const float lr = 0.1f;
    for (int it = 0; it < 200; ++it)
    {
        w.clear_grad();
        b.clear_grad();
        auto pred = F::mat_mul(x, w) + F::broadcast_to(b, Shape{n, 1});
        auto diff = pred - y;
        auto loss = F::sum(diff * diff) * (1.0f / n);
        loss.backward();
        odl_check(odl_axpy(-lr, w.grad().data_ptr<float>(), w.data_ptr<float>(), 1, nullptr));
        odl_check(odl_axpy(-lr, b.grad().data_ptr<float>(), b.data_ptr<float>(), 1, nullptr));
    }
    EXPECT_NEAR(w.item<float>(), 2.0f, 0.1f);
    EXPECT_NEAR(b.item<float>(), 5.0f, 0.1f);
}
// ---- nn::MLP training through the operator tape equals the composition of its parts
static void mlp_training()
{
    nn::MLP model({8, 16, 4});
    auto named = model.named_parameters("");
    EXPECT_TRUE(named.size() == 4 && named.count("layer_0.weight") && named.count("layer_1.bias"));
    EXPECT_TRUE(named.at("layer_0.weight")->shape() == (Shape{8, 16}) && named.at("layer_0.bias")->shape() == (Shape{1, 16}));
    Adam opt(model, 1e-2f);
    WeightDecay wd(1e-4f);
    opt.register_hook(wd.hook());
    std::mt19937 gen(3);
    std::normal_distribution<float> nd;
    std::vector<float> xv(32 * 8);
    for (auto &v : xv)
        v = nd(gen);
    std::vector<int32_t> tv(32);
    for (size_t i = 0; i < tv.size(); ++i)
        tv[i] = (xv[i * 8] > 0) + 2 * (xv[i * 8 + 1] > 0);  // learnable labels
    auto x = T(xv, {32, 8});
    Tensor t(tv, Shape{32}, dtype(DataType::kInt32));
    float first = 0, last = 0;
    for (int s = 0; s < 60; ++s)
    {
        auto loss = F::softmax_cross_entropy(model(x), t);
        if (s == 0)
            first = loss.item<float>();
        last = loss.item<float>();
        opt.zero_grad();
        loss.backward();
        opt.step();
    }
    EXPECT_NEAR(first, std::log(4.0f), 0.8f);
    EXPECT_TRUE(last < 0.5f * first);
    {
        NoGradGuard g;  // no tape is recorded under no_grad()
        auto out = model(x);
        EXPECT_TRUE(!out.impl()->creator);
    }
}
// ---- tests/unit_test/operator/test_batch_norm.cpp, tests/unit_test/nn/test_batch_norm.cpp (same inputs; the reference
//      only checks shapes and finiteness there -- the values below are the closed forms) and silu
static void batch_norm_cases()
{
    const float eps = 1e-5f;
    // BatchNorm1dForwardTraining: x = [[1,2,3],[4,5,6]] -> mean [2.5,3.5,4.5], biased var 2.25
    auto x1 = T({1, 2, 3, 4, 5, 6}, {2, 3}, true);
    auto g1 = T({1, 1, 1}, {3}, true), b1 = T({0, 0, 0}, {3}, true), rm1 = T({0, 0, 0}, {3}), rv1 = T({1, 1, 1}, {3});
    auto y1 = F::batch_norm(x1, g1, b1, rm1, rv1, true, eps, 0.1f, 2);
    EXPECT_TRUE(y1.shape() == (Shape{2, 3}));
    const float n1 = 1.5f / std::sqrt(2.25f + eps);
    expect_tensor(y1, {-n1, -n1, -n1, n1, n1, n1}, 1e-6f);
    expect_tensor(rm1, {0, 0, 0});  // the functional form leaves the running statistics alone
    // BatchNorm1dForwardEval: running statistics (0, 1)
    auto y1e = F::batch_norm(x1, g1, b1, rm1, rv1, false, eps, 0.1f, 2);
    const float k = 1.0f / std::sqrt(1.0f + eps);
    expect_tensor(y1e, {1 * k, 2 * k, 3 * k, 4 * k, 5 * k, 6 * k}, 1e-6f);
    // BatchNorm1dWithGammaBeta: gamma [2, 3], beta [1, -1]
    auto y1g = F::batch_norm(T({1, 2, 3, 4}, {2, 2}), T({2, 3}, {2}), T({1, -1}, {2}), T({0, 0}, {2}), T({1, 1}, {2}), true,
                             eps, 0.1f, 2);
    const float n2 = 1.0f / std::sqrt(1.0f + eps);
    expect_tensor(y1g, {1 - 2 * n2, -1 - 3 * n2, 1 + 2 * n2, -1 + 3 * n2}, 1e-6f);
    // BatchNorm2dForwardTraining: {2,2,2,2}, channel c of image n holds n*8 + c*4 + {1,2,3,4}
    std::vector<float> xv(16);
    for (int i = 0; i < 16; ++i)
        xv[i] = (float)(i + 1);
    auto x2 = T(xv, {2, 2, 2, 2}, true);
    auto g2 = T({1, 1}, {2}, true), b2 = T({0, 0}, {2}, true);
    auto op = std::make_shared<F::BatchNorm>(true, eps, 0.1f, 4);
    auto y2 = op->call1({x2, g2, b2, T({0, 0}, {2}), T({1, 1}, {2})});
    EXPECT_TRUE(y2.shape() == (Shape{2, 2, 2, 2}));
    expect_tensor(op->mean(), {6.5f, 10.5f}, 1e-6f);    // mean of {1..4, 9..12} and of {5..8, 13..16}
    expect_tensor(op->var(), {17.25f, 17.25f}, 1e-5f);
    EXPECT_NEAR(y2.to_vector<float>()[0], (1.0f - 6.5f) / std::sqrt(17.25f + eps), 1e-6f);
    // backward after a TRAINING forward (the reference's operator throws here): sum(gx) = 0 per channel,
    // dbeta = sum(gy), dgamma = sum(gy * x_norm)
    auto w2 = T({1, -2, 3, 0.5f, 2, 1, -1, 4, 0, 1, 1, -3, 2, 2, -1, 0.25f}, {2, 2, 2, 2});
    F::sum(y2 * w2).backward();
    auto gx = x2.grad().to_vector<float>();
    EXPECT_NEAR(gx[0] + gx[1] + gx[2] + gx[3] + gx[8] + gx[9] + gx[10] + gx[11], 0.0f, 1e-5f);
    expect_tensor(b2.grad(), {1 - 2 + 3 + 0.5f + 0 + 1 + 1 - 3, 2 + 1 - 1 + 4 + 2 + 2 - 1 + 0.25f}, 1e-5f);
    auto yv = y2.to_vector<float>(), wv = w2.to_vector<float>();
    float dg0 = 0.f;
    for (int i : {0, 1, 2, 3, 8, 9, 10, 11})
        dg0 += yv[i] * wv[i];
    EXPECT_NEAR(g2.grad().to_vector<float>()[0], dg0, 1e-5f);
    // invalid inputs (src/mat/origin/cpu/normalization/batch_norm.cpp:29-45)
    EXPECT_THROW(F::batch_norm(x2, g2, b2, T({0, 0}, {2}), T({1, 1}, {2}), true, eps, 0.1f, 2));
    EXPECT_THROW(F::batch_norm(x2, g1, b2, T({0, 0}, {2}), T({1, 1}, {2}), true, eps, 0.1f, 4));
    EXPECT_THROW(F::batch_norm(x1, g1, b1, rm1, rv1, true, eps, 0.1f, 3));
    // nn::BatchNorm2d: BasicForward / EvalMode and the running-statistics rule
    nn::BatchNorm2d bn(2, eps, 0.1f);
    EXPECT_TRUE(bn.is_training());
    auto yb = bn(x2.detach());
    EXPECT_TRUE(yb.shape() == (Shape{2, 2, 2, 2}));
    expect_tensor(bn.running_mean(), {0.9f * 6.5f, 0.9f * 10.5f}, 1e-5f);  // 0.1 * 0 + 0.9 * batch mean
    expect_tensor(bn.running_var(), {0.1f + 0.9f * 17.25f, 0.1f + 0.9f * 17.25f}, 1e-4f);
    bn.eval();
    EXPECT_TRUE(!bn.is_training());
    auto ye = bn(x2.detach());
    EXPECT_NEAR(ye.to_vector<float>()[0], (1.0f - 5.85f) / std::sqrt(15.625f + eps), 1e-5f);
    expect_tensor(bn.running_mean(), {0.9f * 6.5f, 0.9f * 10.5f}, 1e-5f);  // unchanged in evaluation mode
    EXPECT_TRUE(bn.named_parameters("").count("weight") && bn.named_parameters("").count("bias"));
    EXPECT_THROW(bn(x1.detach()));
    EXPECT_THROW(nn::BatchNorm2d(0));
    // fused activation: BatchNorm2d(act = SiLU) == silu(BatchNorm2d)
    nn::BatchNorm2d fused(2, eps, 0.1f, ODL_ACT_SILU), plain(2, eps, 0.1f);
    EXPECT_TRUE(fused(x2.detach()).to_vector<float>() == F::silu(plain(x2.detach())).to_vector<float>());
    // silu values and gradient: silu(0) = 0, silu(1) = 0.7310586, silu'(0) = 0.5
    auto xs = T({0, 1, -1, 4}, {4}, true);
    auto ys = F::silu(xs);
    expect_tensor(ys, {0.0f, 0.7310586f, -0.2689414f, 3.9280552f}, 1e-6f);
    F::sum(ys).backward();
    expect_tensor(xs.grad(), {0.5f, 0.9276706f, 0.0723295f, 1.0526646f}, 1e-6f);
}

// ---- state dict, .odl files, checkpoints (tests/unit_test/io/test_checkpoint.cpp: SaveAndLoadCheckpoint,
//      SaveAndLoadModelStateDict, OptimizerStateDict) plus what the reference cannot do: resume on the same trajectory
static std::string g_golden_dir;  // tests/golden of this repository (argv[1]); empty = skip the fixture cases

static float train_steps(nn::MLP &model, Optimizer &opt, const Tensor &x, const Tensor &t, int n)
{
    float last = 0.f;
    for (int s = 0; s < n; ++s)
    {
        auto loss = F::softmax_cross_entropy(model(x), t);
        last      = loss.item<float>();
        opt.zero_grad();
        loss.backward();
        opt.step();
    }
    return last;
}

static void checkpoint_cases()
{
    namespace fs          = std::filesystem;
    const std::string dir = (fs::temp_directory_path() / ("odl_host_test_" + std::to_string((long long)::getpid()))).string();
    fs::create_directories(dir);
    std::mt19937 gen(5);
    std::normal_distribution<float> nd;
    std::vector<float> xv(16 * 4);
    for (auto &v : xv)
        v = nd(gen);
    std::vector<int32_t> tv(16);
    for (size_t i = 0; i < tv.size(); ++i)
        tv[i] = xv[i * 4] > 0;
    auto x = T(xv, {16, 4});
    Tensor t(tv, Shape{16}, dtype(DataType::kInt32));

    // SaveAndLoadModelStateDict
    {
        nn::MLP model({3, 5, 2});
        StateDict sd = model.state_dict();
        EXPECT_TRUE(sd.size() == 4);
        save(sd, dir + "/test_model.odl");
        EXPECT_TRUE(fs::exists(dir + "/test_model.odl"));
        StateDict back = load(dir + "/test_model.odl");
        EXPECT_TRUE(back.size() == sd.size());
        for (auto &kv : sd)
        {
            EXPECT_TRUE(back.count(kv.first) && back.at(kv.first).shape() == kv.second.shape());
            EXPECT_TRUE(back.at(kv.first).to_vector<float>() == kv.second.to_vector<float>());
        }
        nn::MLP fresh({3, 5, 2});
        fresh.load_state_dict(back);
        auto probe = T({0.5f, -1.0f, 2.0f}, {1, 3});
        EXPECT_TRUE(fresh(probe).to_vector<float>() == model(probe).to_vector<float>());
        EXPECT_TRUE(fresh(probe).shape() == (Shape{1, 2}));
        nn::MLP via_file({3, 5, 2});
        via_file.load(dir + "/test_model.odl");
        EXPECT_TRUE(via_file(probe).to_vector<float>() == model(probe).to_vector<float>());
        // strictness (src/nn/module.cpp:130-168)
        StateDict missing = back;
        missing.erase("layer_1.bias");
        EXPECT_THROW(fresh.load_state_dict(missing));
        fresh.load_state_dict(missing, false);
        StateDict extra = back;
        extra["unknown"] = Tensor::zeros(Shape{1});
        EXPECT_THROW(fresh.load_state_dict(extra));
        StateDict wrong = back;
        wrong["layer_0.weight"] = Tensor::zeros(Shape{5, 3});
        EXPECT_THROW(fresh.load_state_dict(wrong, false));
        EXPECT_THROW(load(dir + "/no_such_file.odl"));
        {
            std::ofstream bad(dir + "/bad.odl", std::ios::binary);
            bad << "not an odl file";
        }
        EXPECT_THROW(load(dir + "/bad.odl"));
    }
    // OptimizerStateDict
    {
        nn::MLP model({2, 4, 1});
        Adam optimizer(model, 0.01f, 0.9f, 0.999f, 1e-8f);
        auto st = optimizer.state_dict();
        EXPECT_TRUE(st.count("lr") && st.count("beta1") && st.count("beta2") && st.count("eps"));
        EXPECT_TRUE(std::any_cast<float>(st.at("lr")) == 0.01f && std::any_cast<float>(st.at("beta1")) == 0.9f);
        EXPECT_TRUE(std::any_cast<float>(st.at("beta2")) == 0.999f && std::any_cast<float>(st.at("eps")) == 1e-8f);
        EXPECT_TRUE(std::any_cast<StateDict>(st.at("m_buffers")).empty());  // no step taken yet
    }
    // SaveAndLoadCheckpoint, and resuming: Adam moments and step counts travel, so the run continues bit for bit
    {
        nn::MLP model({4, 8, 2});
        Adam optimizer(model, 0.001f);
        train_steps(model, optimizer, x, t, 5);
        Checkpoint ck;
        ck.model_state_dict             = model.state_dict();
        ck.optimizer_state_dict["adam"] = optimizer.state_dict();
        ck.epoch                        = 5;
        ck.step                         = 100;
        ck.loss                         = 0.5f;
        ck.optimizer_type               = "Adam";
        ck.optimizer_config["lr"]       = 0.001f;
        ck.optimizer_config["beta1"]    = 0.9f;
        ck.optimizer_config["beta2"]    = 0.999f;
        ck.optimizer_config["eps"]      = 1e-8f;
        const std::string path          = dir + "/test_checkpoint.ckpt";
        save(ck, path);
        EXPECT_TRUE(fs::exists(dir + "/test_checkpoint") && fs::exists(dir + "/test_checkpoint/model.odl"));
        EXPECT_TRUE(fs::exists(dir + "/test_checkpoint/metadata.json") && fs::exists(dir + "/test_checkpoint/optimizer.odl"));
        Checkpoint back = load_checkpoint(path);
        EXPECT_TRUE(back.epoch == 5 && back.step == 100 && back.loss == 0.5f && back.optimizer_type == "Adam");
        EXPECT_NEAR(back.optimizer_config.at("lr"), 0.001f, 1e-9f);
        EXPECT_NEAR(back.optimizer_config.at("beta1"), 0.9f, 1e-7f);
        EXPECT_NEAR(back.optimizer_config.at("beta2"), 0.999f, 1e-7f);
        EXPECT_NEAR(back.optimizer_config.at("eps"), 1e-8f, 1e-14f);
        EXPECT_TRUE(back.model_state_dict.size() == ck.model_state_dict.size());
        const float next_a = train_steps(model, optimizer, x, t, 4);

        nn::MLP resumed({4, 8, 2});
        resumed.load_state_dict(back.model_state_dict);
        Adam optimizer_b(resumed, 0.5f);  // configuration comes from the checkpoint
        EXPECT_TRUE(back.optimizer_state_dict.count("adam") == 1);
        optimizer_b.load_state_dict(back.optimizer_state_dict.at("adam"));
        auto steps = std::any_cast<std::unordered_map<std::string, int>>(optimizer_b.state_dict().at("step_counts"));
        EXPECT_TRUE(steps.size() == 4 && steps.at("step_layer_0.weight") == 5);
        const float next_b = train_steps(resumed, optimizer_b, x, t, 4);
        EXPECT_TRUE(next_a == next_b);
        for (auto &kv : model.state_dict())
            EXPECT_TRUE(resumed.state_dict().at(kv.first).to_vector<float>() == kv.second.to_vector<float>());
        EXPECT_THROW(load_checkpoint(dir + "/absent.ckpt"));
    }
    // SGD momentum buffers through the same path
    {
        nn::MLP model({4, 8, 2});
        SGD optimizer(model, 0.05f, 0.9f);
        train_steps(model, optimizer, x, t, 3);
        Checkpoint ck;
        ck.model_state_dict            = model.state_dict();
        ck.optimizer_state_dict["sgd"] = optimizer.state_dict();
        ck.optimizer_type              = "SGD";
        ck.optimizer_config["lr"]      = 0.05f;
        save(ck, dir + "/sgd.ckpt");
        const float next_a = train_steps(model, optimizer, x, t, 3);
        Checkpoint back    = load_checkpoint(dir + "/sgd.ckpt");
        nn::MLP resumed({4, 8, 2});
        resumed.load_state_dict(back.model_state_dict);
        SGD optimizer_b(resumed, 0.05f, 0.9f);
        optimizer_b.load_state_dict(back.optimizer_state_dict.at("sgd"));
        EXPECT_TRUE(train_steps(resumed, optimizer_b, x, t, 3) == next_a);
    }
    // files written by the unmodified reference (tests/golden/make_odl_fixtures.py)
    if (!g_golden_dir.empty())
    {
        StateDict sd = load(g_golden_dir + "/ref_state.odl");
        EXPECT_TRUE(sd.size() == 4 && sd.at("conv.weight").shape() == (Shape{2, 3, 2, 2}) && sd.at("head.scale").shape() == (Shape{7}));
        EXPECT_TRUE(sd.at("layer_0.weight").shape() == (Shape{3, 5}) && sd.at("layer_0.bias").shape() == (Shape{1, 5}));
        Checkpoint ck = load_checkpoint(g_golden_dir + "/ref_checkpoint.ckpt");
        EXPECT_TRUE(ck.epoch == 5 && ck.step == 100 && ck.loss == 0.5f && ck.optimizer_type == "Adam");
        EXPECT_TRUE(ck.optimizer_state_dict.empty());  // the reference writes no optimizer.odl
        nn::MLP model({4, 8, 2});
        model.load_state_dict(ck.model_state_dict);
        EXPECT_TRUE(model(x).shape() == (Shape{16, 2}));
        // saved again by this layer, the file holds the same records (sorted by name here, hash order there)
        save(ck.model_state_dict, dir + "/resaved.odl");
        EXPECT_TRUE(fs::file_size(dir + "/resaved.odl") == fs::file_size(g_golden_dir + "/ref_checkpoint/model.odl"));
    }
    fs::remove_all(dir);
}

// ---- memory pool: bins and reuse (src/mat/origin/memory/memory_pool.cpp)
// ---- DataLoader: the cases of tests/unit_test/data/test_dataloader.cpp (BasicIteration, Reset, Shuffle, BatchSizeOne,
//      EmptyDataset) plus the VALUES of every batch, integer labels (int64 out), multi-element samples, the uncached mode
//      and training straight from the loader.
namespace
{
class IndexDataset : public Dataset
{
  public:
    IndexDataset(size_t n, size_t width, bool int_labels) : n_(n), width_(width), int_labels_(int_labels) {}
    std::pair<Tensor, Tensor> get_item(size_t index) override
    {
        if (index >= n_)
            throw std::out_of_range("Index out of range");
        ++calls;
        std::vector<float> v(width_);
        for (size_t j = 0; j < width_; ++j)
            v[j] = static_cast<float>(index) + 0.25f * static_cast<float>(j);
        Tensor x = width_ == 4 ? Tensor(v, Shape{2, 2}) : Tensor(v, Shape{width_});
        Tensor t = int_labels_ ? Tensor(std::vector<int32_t>{static_cast<int32_t>(index % 10)}, Shape{}, dtype(DataType::kInt32))
                               : Tensor(std::vector<float>{static_cast<float>(index % 10)}, Shape{});
        return {x, t};
    }
    size_t size() const override { return n_; }
    size_t calls = 0;

  private:
    size_t n_, width_;
    bool int_labels_;
};
}  // namespace

static void dataloader_cases()
{
    {  // BasicIteration: 10 samples in batches of 3 -> 3, 3, 3, 1; values follow the index order
        IndexDataset ds(10, 1, false);
        DataLoader loader(ds, 3, false);
        EXPECT_TRUE(loader.has_next() && loader.batch_size() == 3 && loader.dataset_size() == 10);
        size_t seen = 0;
        for (size_t want : {3u, 3u, 3u, 1u})
        {
            auto [x, t] = loader.next();
            EXPECT_TRUE(x.shape() == Shape({want, 1}) && t.shape() == Shape({want}) && t.dtype() == DataType::kFloat32);
            auto xv = x.to_vector<float>(), tv = t.to_vector<float>();
            for (size_t i = 0; i < want; ++i, ++seen)
                EXPECT_TRUE(xv[i] == static_cast<float>(seen) && tv[i] == static_cast<float>(seen % 10));
        }
        EXPECT_TRUE(!loader.has_next());
        EXPECT_THROW(loader.next());
        EXPECT_TRUE(ds.calls == 10);  // the data set was read once
    }
    {  // Reset
        IndexDataset ds(5, 1, false);
        DataLoader loader(ds, 2, false);
        loader.next();
        EXPECT_TRUE(loader.has_next());
        loader.reset();
        auto [x, t] = loader.next();
        EXPECT_TRUE(x.shape()[0] == 2 && x.to_vector<float>()[0] == 0.0f);
    }
    {  // Shuffle: a permutation, reproducible for one seed, different after reset(); int32 labels come out as int64
        IndexDataset ds(50, 4, true);
        DataLoader a(ds, 50, true, 7), b(ds, 50, true, 7);
        auto [xa, ta] = a.next();
        auto [xb, tb] = b.next();
        EXPECT_TRUE(xa.shape() == Shape({50, 4}) && ta.dtype() == DataType::kInt64);
        auto va = xa.to_vector<float>(), vb = xb.to_vector<float>();
        auto la = ta.to_vector<int64_t>();
        EXPECT_TRUE(va == vb);
        std::vector<int> hit(50, 0);
        bool in_order = true, rows_ok = true;
        for (size_t i = 0; i < 50; ++i)
        {
            const int id = static_cast<int>(va[4 * i]);
            hit[id]++;
            in_order = in_order && id == static_cast<int>(i);
            rows_ok  = rows_ok && va[4 * i + 3] == static_cast<float>(id) + 0.75f && la[i] == id % 10;
        }
        EXPECT_TRUE(rows_ok && !in_order && *std::min_element(hit.begin(), hit.end()) == 1);
        a.reset();
        EXPECT_TRUE(a.next().first.to_vector<float>() != va);
    }
    {  // BatchSizeOne
        IndexDataset ds(5, 1, false);
        DataLoader loader(ds, 1, false);
        for (size_t i = 0; i < 5; ++i)
        {
            EXPECT_TRUE(loader.has_next());
            auto [x, t] = loader.next();
            EXPECT_TRUE(x.shape()[0] == 1 && t.shape()[0] == 1 && x.to_vector<float>()[0] == static_cast<float>(i));
        }
        EXPECT_TRUE(!loader.has_next());
    }
    {  // EmptyDataset
        IndexDataset ds(0, 1, false);
        DataLoader loader(ds, 1, false);
        EXPECT_TRUE(!loader.has_next() && loader.dataset_size() == 0);
        EXPECT_THROW(loader.next());
    }
    {  // uncached mode: get_item() runs for every sample of every epoch, batches are the same
        IndexDataset ds(7, 4, true);
        DataLoader cached(ds, 3, false), fresh(ds, 3, false, 0, false);
        while (cached.has_next())
        {
            auto c = cached.next();
            auto f = fresh.next();
            EXPECT_TRUE(c.first.to_vector<float>() == f.first.to_vector<float>() &&
                        c.second.to_vector<int64_t>() == f.second.to_vector<int64_t>());
        }
        EXPECT_TRUE(!fresh.has_next());
        const size_t before = ds.calls;
        fresh.reset();
        while (fresh.has_next())
            fresh.next();
        EXPECT_TRUE(ds.calls == before + 7);
    }
    {  // training from the loader: the loss of a small classifier falls
        IndexDataset ds(64, 4, true);
        DataLoader loader(ds, 16, true, 3);
        nn::MLP model({4, 32, 10});
        Adam opt(model, 1e-2f);
        float first = 0.f, last = 0.f;
        for (int epoch = 0; epoch < 30; ++epoch)
        {
            loader.reset();
            while (loader.has_next())
            {
                auto [x, t] = loader.next();
                Tensor loss = functional::softmax_cross_entropy(model(x), t);
                model.zero_grad();
                loss.backward();
                opt.step();
                last = loss.item<float>();
                if (epoch == 0 && first == 0.f)
                    first = last;
            }
        }
        EXPECT_TRUE(last < 0.7f * first);
    }
}

// ---- Sequential of the layers of the reference's CNN example (conv -> BatchNorm2d -> ReLU -> conv -> Flatten -> Linear):
//      against the same chain written with the functional API on the SAME parameters, gradients included; state dict
//      names; error cases of Sequential::operator[] and flatten (tests/unit_test/nn/test_sequential.cpp style).
static void sequential_cnn()
{
    Sequential net;
    net.add(std::make_unique<nn::Conv2d>(3, 8, 3, 1, 1));
    net.add(std::make_unique<nn::BatchNorm2d>(8));
    net.add(std::make_unique<nn::ReLU>());
    net.add(std::make_unique<nn::Conv2d>(8, 6, 3, 2, 1));
    net.add(std::make_unique<nn::Flatten>());
    net.add(std::make_unique<nn::Linear>(6 * 5 * 6, 5));
    EXPECT_TRUE(net.size() == 6);
    EXPECT_THROW(net[6]);
    EXPECT_TRUE(net.parameters().size() == 8);
    auto sd = net.state_dict();
    EXPECT_TRUE(sd.size() == 8 && sd.count("0.weight") && sd.count("1.bias") && sd.count("3.bias") && sd.count("5.weight"));

    Tensor x = Tensor::randn(Shape{4, 3, 10, 12}, TensorOptions(), 11);
    Tensor t(std::vector<int32_t>{0, 3, 1, 4}, Shape{4}, dtype(DataType::kInt32));
    Tensor y = net(x);
    EXPECT_TRUE(y.shape() == Shape({4, 5}));
    Tensor loss = functional::softmax_cross_entropy(y, t);
    net.zero_grad();
    loss.backward();
    std::vector<std::vector<float>> grads;
    for (Parameter *p : net.parameters())
        grads.push_back(p->grad().to_vector<float>());

    // the same chain through the functional API
    auto &c1 = static_cast<nn::Conv2d &>(net[0]);
    auto &bn = static_cast<nn::BatchNorm2d &>(net[1]);
    auto &c2 = static_cast<nn::Conv2d &>(net[3]);
    auto &fc = static_cast<nn::Linear &>(net[5]);
    Tensor rm = Tensor::zeros(Shape{8}), rv = Tensor::ones(Shape{8});
    Tensor h  = functional::conv2d(x, *c1.weight(), c1.bias(), 1, 1);
    h         = functional::batch_norm(h, *bn.weight(), *bn.bias(), rm, rv, true);
    h         = functional::relu(h);
    h         = functional::conv2d(h, *c2.weight(), c2.bias(), 2, 1);
    h         = functional::flatten(h);
    EXPECT_TRUE(h.shape() == Shape({4, 180}));
    h          = fc(h);
    expect_tensor(h, y.to_vector<float>(), 1e-6f);
    Tensor loss2 = functional::softmax_cross_entropy(h, t);
    net.zero_grad();
    loss2.backward();
    size_t i = 0;
    for (Parameter *p : net.parameters())
        expect_tensor(p->grad(), grads[i++], 1e-6f);

    // flatten / reshape: shapes, errors, gradient shape
    Tensor z = Tensor::randn(Shape{2, 3, 4, 5}, TensorOptions().requires_grad(true), 5);
    EXPECT_TRUE(functional::flatten(z, 1, 2).shape() == Shape({2, 12, 5}));
    EXPECT_TRUE(functional::flatten(z, 0, -1).shape() == Shape({120}));
    EXPECT_THROW(functional::flatten(z, 2, 1));
    EXPECT_THROW(functional::flatten(z, 0, 4));
    EXPECT_THROW(functional::reshape(z, Shape{7, 7}));
    Tensor s = functional::sum(functional::flatten(z) * 2.0f);
    s.backward();
    EXPECT_TRUE(z.grad().shape() == z.shape());
    expect_tensor(z.grad(), std::vector<float>(120, 2.0f), 0.f);

    // it trains: evaluation mode uses the running statistics the training steps produced
    SGD opt(net, 0.05f);
    float first = 0.f, last = 0.f;
    for (int step = 0; step < 40; ++step)
    {
        Tensor l = functional::softmax_cross_entropy(net(x), t);
        net.zero_grad();
        l.backward();
        opt.step();
        last = l.item<float>();
        if (step == 0)
            first = last;
    }
    EXPECT_TRUE(last < 0.5f * first);
    net.eval();
    EXPECT_TRUE(net(x).shape() == Shape({4, 5}) && !net[1].is_training());
    EXPECT_THROW(nn::Conv2d(3, 8, {3, 3}, {1, 2}));
    EXPECT_THROW(nn::Conv2d(0, 8, 3));
}

// ---- The fused, device-resident MLP trainer of the C ABI driven from C++: eager steps (odl_mlp_train_step) against the
//      whole-step CUDA graph recorded by the library (odl_mlp_capture / odl_mlp_replay) -- same losses, same parameters.
static void mlp_graph_step()
{
    const int32_t sizes[] = {64, 96, 48, 10};
    const int64_t batch   = 32;
    void *eager = nullptr, *graphed = nullptr;
    odl_check(odl_mlp_create(sizes, 4, batch, 1, 1e-3f, 0.f, 1e-4f, ODL_PRECISION_3XTF32, &eager));
    odl_check(odl_mlp_create(sizes, 4, batch, 1, 1e-3f, 0.f, 1e-4f, ODL_PRECISION_3XTF32, &graphed));
    const int64_t n = odl_mlp_param_count(eager);
    std::vector<float> p0(n);
    std::mt19937 gen(3);
    std::normal_distribution<float> nd(0.f, 0.1f);
    for (auto &v : p0)
        v = nd(gen);
    odl_check(odl_mlp_set_params(eager, p0.data(), nullptr));
    odl_check(odl_mlp_set_params(graphed, p0.data(), nullptr));
    Tensor x = Tensor::randn(Shape{(size_t)batch, 64}, TensorOptions(), 9);
    std::vector<int32_t> lab(batch);
    for (int i = 0; i < batch; ++i)
        lab[i] = i % 10;
    Tensor t(lab, Shape{(size_t)batch}, dtype(DataType::kInt32));
    synchronize();
    cudaStream_t stream;
    cuda_check(cudaStreamCreate(&stream), "stream");
    odl_check(odl_mlp_capture(graphed, x.data_ptr<float>(), t.data_ptr<void>(), 0, stream));
    EXPECT_TRUE(odl_mlp_step_count(graphed) == 0);  // recording takes no optimisation step
    float le = 0.f, lg = 0.f;
    for (int step = 0; step < 5; ++step)
    {
        odl_check(odl_mlp_train_step(eager, x.data_ptr<float>(), t.data_ptr<void>(), 0, stream));
        cuda_check(cudaMemcpyAsync(&le, odl_mlp_loss_ptr(eager), 4, cudaMemcpyDeviceToHost, stream), "loss");
        odl_check(odl_mlp_replay(graphed, stream));
        cuda_check(cudaMemcpyAsync(&lg, odl_mlp_loss_ptr(graphed), 4, cudaMemcpyDeviceToHost, stream), "loss");
        cuda_check(cudaStreamSynchronize(stream), "sync");
        EXPECT_TRUE(le == lg && std::isfinite(le));
    }
    std::vector<float> pe(n), pg(n);
    odl_check(odl_mlp_get_packed(eager, 0, pe.data(), stream));
    odl_check(odl_mlp_get_packed(graphed, 0, pg.data(), stream));
    cuda_check(cudaStreamSynchronize(stream), "sync");
    EXPECT_TRUE(pe == pg && odl_mlp_step_count(graphed) == 5);
    EXPECT_TRUE(odl_mlp_capture(graphed, x.data_ptr<float>(), t.data_ptr<void>(), 0, nullptr) != 0);  // default stream refused
    odl_check(odl_mlp_destroy(eager));
    odl_check(odl_mlp_destroy(graphed));
    cudaStreamDestroy(stream);
}

static void memory_pool()
{
    EXPECT_TRUE(MemoryPool::bin_size(1) == 256 && MemoryPool::bin_size(257) == 512 && MemoryPool::bin_size(300000) == 524288);
    EXPECT_TRUE(MemoryPool::bin_size(600000) == (1u << 20) && MemoryPool::bin_size(3u << 20) == (4u << 20));
    EXPECT_TRUE(MemoryPool::bin_size(17u << 20) == (32u << 20));
    auto &pool        = MemoryPool::instance();
    const size_t hits = pool.hits();
    void *p1          = nullptr;
    {
        Tensor a = Tensor::zeros(Shape{1000});
        p1       = a.data_ptr<float>();
    }
    Tensor b = Tensor::zeros(Shape{1000});
    EXPECT_TRUE(b.data_ptr<float>() == p1 && pool.hits() > hits);  // the freed block was handed out again
}

int main(int argc, char **argv)
{
    if (argc > 1)
        g_golden_dir = argv[1];
    try
    {
        init(0);
    }
    catch (const std::exception &e)
    {
        std::printf("cannot initialise: %s\n", e.what());
        return 2;
    }
    const std::vector<std::pair<const char *, std::function<void()>>> tests = {
        {"matmul_forward", matmul_forward},   {"matmul_backward", matmul_backward},
        {"linear_forward", linear_forward},   {"linear_backward", linear_backward},
        {"relu", relu_cases},                 {"softmax_cross_entropy", softmax_ce_cases},
        {"conv2d", conv2d_cases},             {"weight_decay_and_adam", weight_decay_and_adam},
        {"linear_regression", linear_regression}, {"mlp_training", mlp_training},
        {"memory_pool", memory_pool},         {"checkpoint", checkpoint_cases},
        {"batch_norm_silu", batch_norm_cases},
        {"dataloader", dataloader_cases},     {"sequential_cnn", sequential_cnn},
        {"mlp_graph_step", mlp_graph_step}};
    for (auto &t : tests)
    {
        const int before = g_failed;
        try
        {
            t.second();
            synchronize();
        }
        catch (const std::exception &e)
        {
            ++g_failed;
            std::printf("    EXCEPTION in %s: %s\n", t.first, e.what());
        }
        std::printf("[%s] %s\n", g_failed == before ? "  OK  " : "FAILED", t.first);
    }
    std::printf("%d checks, %d failed\n", g_checks, g_failed);
    return g_failed ? 1 : 0;
}
