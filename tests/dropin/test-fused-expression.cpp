// The reference's expression templates evaluated as one kernel (fused.hpp) against their own
// node-by-node forward(), on the device, through the unmodified front-end.
#ifdef CUDA
#include <gtest/gtest.h>

#include "tensor.hpp"
#include "comparisons.hpp"
#include "functions.hpp"

#include "fused.hpp"

using namespace tannic;

static Tensor ramp(type dtype, Shape shape, float from, float step) {
    Tensor t(dtype, shape);
    t.initialize(Device());
    size_t n = 1;
    for (auto s : shape) n *= s;
    std::vector<float> host(n);
    for (size_t i = 0; i < n; ++i) host[i] = from + step * static_cast<float>(i % 97);
    // one bulk copy instead of one per element
    tn_device_t d{0};
    tn_copy_from_host(&d, host.data(), t.bytes(), n * sizeof(float));
    return t;
}

TEST(FusedExpression, OneLaunchForTheWholeTree) {
    Tensor X = ramp(float32, {64, 256}, 0.25f, 0.03f);
    Tensor Y = ramp(float32, {1, 256}, -1.5f, 0.04f);
    auto tree = log(X) + Y * Y - exp(X);
    const uint64_t before = tn_launch_count();
    Tensor Z = b200::fused(tree);
    EXPECT_EQ(tn_launch_count() - before, 1u);
    Tensor chain = tree.forward(Context{});  // five kernels, four temporaries
    EXPECT_EQ(tn_launch_count() - before, 6u);
    EXPECT_TRUE(allclose(Z, chain, 1e-5, 1e-6));
}

TEST(FusedExpression, ScalarsFunctionsAndSharedOperands) {
    Tensor X = ramp(float32, {32, 128}, 0.5f, 0.02f);
    Tensor W = ramp(float32, {32, 128}, -0.7f, 0.015f);
    Tensor B = ramp(float32, {128}, 0.1f, 0.01f);
    auto tree = tanh(X * W + B) * 0.5f - rsqrt(X, 1e-5f);
    const uint64_t before = tn_launch_count();
    Tensor Z = b200::fused(tree);
    EXPECT_EQ(tn_launch_count() - before, 1u);
    EXPECT_TRUE(allclose(Z, tree.forward(Context{}), 1e-5, 1e-6));
}

TEST(FusedExpression, FallsBackWhenTheTreeDoesNotFit) {
    Tensor A = ramp(float32, {8, 8}, 0.0f, 1.0f);
    Tensor H(float32, {8, 8});
    H.initialize();  // host tensor
    auto mixed = A + A;
    Tensor five[5] = {ramp(float32, {4}, 0, 1), ramp(float32, {4}, 1, 1), ramp(float32, {4}, 2, 1), ramp(float32, {4}, 3, 1), ramp(float32, {4}, 4, 1)};
    auto many = five[0] + five[1] + five[2] + five[3] + five[4];  // five distinct tensors: evaluated node by node
    const uint64_t before = tn_launch_count();
    Tensor S = b200::fused(many);
    EXPECT_EQ(tn_launch_count() - before, 4u);
    EXPECT_TRUE(allclose(S, many.forward(Context{})));
    auto host_tree = H + H;
    Tensor R = b200::fused(host_tree);  // host operands: the reference's CPU path
    EXPECT_TRUE(allclose(R, host_tree.forward(Context{})));
    EXPECT_TRUE(allclose(b200::fused(mixed), mixed.forward(Context{})));
}
#endif
