// LinearOp::backward -- the rule the reference leaves unimplemented (src/operators/custom/linear.cpp:116-121) -- tested
// in the reference's own idiom (its gtest base class, both devices): a hand-computed case, and a seeded case where the
// fused operator must give the gradients of the same function written with the reference's unfused operators
// (mat_mul, transpose, broadcast_to, +), whose backward rules the reference does implement.
#include <gtest/gtest.h>

#include <cstdint>
#include <vector>

#include "../common/device_test_base.h"
#include "../common/gtest_utils.h"
#include "../common/test_utils.h"
#include "origin.h"
#include "origin/operators/custom/linear.h"

using namespace origin;
namespace F = origin::functional;

class LinearBackwardTest : public origin::test::OperatorTestBase
{
protected:
    TensorOptions grad_opts() const { return dtype(DataType::kFloat32).device(deviceType()).requires_grad(true); }
    TensorOptions opts() const { return dtype(DataType::kFloat32).device(deviceType()); }
    static std::vector<float> seeded(size_t n, uint32_t seed)
    {
        std::vector<float> v(n);
        uint32_t s = seed * 2654435761u + 12345u;
        for (auto &e : v)
        {
            s = s * 1664525u + 1013904223u;
            e = static_cast<float>(static_cast<int32_t>(s >> 8) % 2001 - 1000) / 500.0f;  // [-2, 2], exact in fp32
        }
        return v;
    }
};

TEST_P(LinearBackwardTest, HandComputed)
{
    // x [2,3], W [2,3] (out, in), b [2]; loss = sum(y)  ->  gy = ones
    auto x = Tensor({1.0f, 2.0f, 3.0f, 4.0f, 5.0f, 6.0f}, Shape{2, 3}, grad_opts());
    auto w = Tensor({1.0f, 0.0f, -1.0f, 2.0f, 1.0f, 0.0f}, Shape{2, 3}, grad_opts());
    auto b = Tensor({0.5f, -0.5f}, Shape{2}, grad_opts());
    auto y = F::custom_linear(x, w, b, 3, 2, true);
    origin::test::GTestUtils::EXPECT_TENSORS_EQ(y, Tensor({-1.5f, 3.5f, -1.5f, 12.5f}, Shape{2, 2}, opts()),
                                                origin::test::TestTolerance::kDefault);
    y.backward();
    // gx = gy . W = [1,1] . [[1,0,-1],[2,1,0]] = [3,1,-1] per row; gW = gy^T . x = column sums of x per output; gb = [2,2]
    origin::test::GTestUtils::EXPECT_TENSORS_EQ(x.grad(), Tensor({3.0f, 1.0f, -1.0f, 3.0f, 1.0f, -1.0f}, Shape{2, 3}, opts()),
                                                origin::test::TestTolerance::kDefault);
    origin::test::GTestUtils::EXPECT_TENSORS_EQ(w.grad(), Tensor({5.0f, 7.0f, 9.0f, 5.0f, 7.0f, 9.0f}, Shape{2, 3}, opts()),
                                                origin::test::TestTolerance::kDefault);
    origin::test::GTestUtils::EXPECT_TENSORS_EQ(b.grad(), Tensor({2.0f, 2.0f}, Shape{2}, opts()),
                                                origin::test::TestTolerance::kDefault);
}

TEST_P(LinearBackwardTest, EqualsTheUnfusedGraph)
{
    const size_t M = 37, K = 130, N = 65;  // ragged on purpose: no multiple of any tile
    const auto xd = seeded(M * K, 1), wd = seeded(N * K, 2), bd = seeded(N, 3), cd = seeded(M * N, 4);
    auto coef = Tensor(cd, Shape{M, N}, opts());  // loss = sum(y * coef)  ->  gy = coef, not constant

    auto x1 = Tensor(xd, Shape{M, K}, grad_opts());
    auto w1 = Tensor(wd, Shape{N, K}, grad_opts());
    auto b1 = Tensor(bd, Shape{N}, grad_opts());
    auto y1 = F::custom_linear(x1, w1, b1, (int)K, (int)N, true);
    auto l1 = F::sum(y1 * coef);
    l1.backward();

    auto x2 = Tensor(xd, Shape{M, K}, grad_opts());
    auto w2 = Tensor(wd, Shape{N, K}, grad_opts());
    // ({1, N} like nn::Linear's bias: the reference's sum_to cannot reduce {M, N} to a 1-D {N} when M != N)
    auto b2 = Tensor(bd, Shape{1, N}, grad_opts());
    auto y2 = F::mat_mul(x2, F::transpose(w2)) + F::broadcast_to(b2, Shape{M, N});
    auto l2 = F::sum(y2 * coef);
    l2.backward();

    origin::test::GTestUtils::EXPECT_TENSORS_NEAR(y1, y2, 1e-5, 1e-4);
    origin::test::GTestUtils::EXPECT_TENSORS_NEAR(x1.grad(), x2.grad(), 1e-5, 1e-4);
    origin::test::GTestUtils::EXPECT_TENSORS_NEAR(w1.grad(), w2.grad(), 1e-5, 1e-4);
    origin::test::GTestUtils::EXPECT_TENSORS_NEAR(b1.grad(), b2.grad().reshape(Shape{N}), 1e-5, 1e-4);
}

TEST_P(LinearBackwardTest, WithoutBiasAndFlattenedInput)
{
    const size_t B = 5, C = 3, H = 4, N = 7, K = C * H;
    const auto xd = seeded(B * K, 5), wd = seeded(N * K, 6);
    auto x = Tensor(xd, Shape{B, C, H}, grad_opts());
    auto w = Tensor(wd, Shape{N, K}, grad_opts());
    auto y = F::custom_linear(x, w, (int)K, (int)N);
    y.backward();
    EXPECT_EQ(x.grad().shape(), (Shape{B, C, H}));  // the gradient has the shape of the input, not of its flattening
    auto x2 = Tensor(xd, Shape{B, K}, grad_opts());
    auto w2 = Tensor(wd, Shape{N, K}, grad_opts());
    auto y2 = F::mat_mul(x2, F::transpose(w2));
    y2.backward();
    origin::test::GTestUtils::EXPECT_TENSORS_NEAR(x.grad().reshape(Shape{B, K}), x2.grad(), 1e-5, 1e-4);
    origin::test::GTestUtils::EXPECT_TENSORS_NEAR(w.grad(), w2.grad(), 1e-5, 1e-4);
}

INSTANTIATE_DEVICE_TEST_SUITE_P(LinearBackwardTest);
