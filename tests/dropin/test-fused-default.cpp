// Fusion as the DEFAULT path: compiled against the header overlay (make_overlay.py) with
// -DTANNIC_B200_FUSE, a plain `Tensor Z = log(X) + Y * Y - exp(X);` through the reference's own
// front-end is one kernel launch, with the values of the node-by-node chain.
#ifdef CUDA
#include <gtest/gtest.h>

#include <cstring>
#include <vector>

#include "tensor.hpp"
#include "comparisons.hpp"
#include "functions.hpp"

#include "fused.hpp"

using namespace tannic;

static Tensor ramp(type dtype, Shape shape, float from, float step, Environment environment = Device()) {
    Tensor t(dtype, shape);
    t.initialize(environment);
    size_t n = 1;
    for (auto s : shape) n *= s;
    std::vector<float> host(n);
    for (size_t i = 0; i < n; ++i) host[i] = from + step * static_cast<float>(i % 97);
    if (std::holds_alternative<Device>(environment)) {
        tn_device_t d{0};
        tn_copy_from_host(&d, host.data(), t.bytes(), n * sizeof(float));
    } else {
        std::memcpy(t.bytes(), host.data(), n * sizeof(float));
    }
    return t;
}

// Device result -> host tensor through the backend's copy (Tensor::to(Host()) of the reference takes the
// device id from the HOST tensor's record, src/tensor.cpp:112-121, so it is not used here).
static Tensor to_host(Tensor const& device_tensor) {
    Tensor host(device_tensor.dtype(), device_tensor.shape());
    host.initialize(Host());
    tn_device_t d{0};
    if (tn_copy_to_host(&d, device_tensor.bytes(), host.bytes(), device_tensor.nbytes()) != TN_SUCCESS) throw std::runtime_error(tn_last_error());
    return host;
}

TEST(FusedByDefault, PlainAssignmentIsOneLaunch) {
    Tensor X = ramp(float32, {64, 256}, 0.25f, 0.03f);
    Tensor Y = ramp(float32, {1, 256}, -1.5f, 0.04f);
    const uint64_t before = tn_launch_count();
    Tensor Z = log(X) + Y * Y - exp(X);  // no helper: the front-end's own forward()
    EXPECT_EQ(tn_launch_count() - before, 1u);
    Tensor XH = ramp(float32, {64, 256}, 0.25f, 0.03f, Host());
    Tensor YH = ramp(float32, {1, 256}, -1.5f, 0.04f, Host());
    Tensor ZH = log(XH) + YH * YH - exp(XH);  // host tensors: the CPU kernels, node by node
    EXPECT_TRUE(allclose(to_host(Z), ZH, 1e-5, 1e-6));
}

TEST(FusedByDefault, ScalarsFunctionsAndSubtreesThatDoNotFit) {
    Tensor X = ramp(float32, {32, 128}, 0.5f, 0.02f);
    Tensor W = ramp(float32, {32, 128}, -0.7f, 0.015f);
    Tensor B = ramp(float32, {128}, 0.1f, 0.01f);
    uint64_t before = tn_launch_count();
    Tensor Z = tanh(X * W + B) * 0.5f - rsqrt(X, 1e-5f);
    EXPECT_EQ(tn_launch_count() - before, 1u);
    EXPECT_TRUE(allclose(Z, b200::fused(tanh(X * W + B) * 0.5f - rsqrt(X, 1e-5f)), 1e-6, 1e-7));
    // a single node keeps the front-end's own path (one launch either way)
    before = tn_launch_count();
    Tensor S = X + W;
    EXPECT_EQ(tn_launch_count() - before, 1u);
    // five distinct tensors do not fit one program: the four-tensor prefix is fused, the last add is its own launch
    Tensor five[5] = {ramp(float32, {4}, 0, 1), ramp(float32, {4}, 1, 1), ramp(float32, {4}, 2, 1), ramp(float32, {4}, 3, 1), ramp(float32, {4}, 4, 1)};
    before = tn_launch_count();
    Tensor T = five[0] + five[1] + five[2] + five[3] + five[4];
    EXPECT_EQ(tn_launch_count() - before, 2u);
    Tensor H[5] = {ramp(float32, {4}, 0, 1, Host()), ramp(float32, {4}, 1, 1, Host()), ramp(float32, {4}, 2, 1, Host()), ramp(float32, {4}, 3, 1, Host()),
                   ramp(float32, {4}, 4, 1, Host())};
    Tensor TH = H[0] + H[1] + H[2] + H[3] + H[4];
    EXPECT_TRUE(allclose(to_host(T), TH));
}

TEST(FusedByDefault, ViewsAndMixedDtypesTakeTheNodeByNodePath) {
    Tensor X = ramp(float32, {8, 8}, 0.0f, 1.0f);
    Tensor V = X.transpose(0, 1);  // strided view: not a program input
    const uint64_t before = tn_launch_count();
    Tensor Z = V + V - X;
    EXPECT_GE(tn_launch_count() - before, 2u);
    Tensor XH = ramp(float32, {8, 8}, 0.0f, 1.0f, Host());
    Tensor VH = XH.transpose(0, 1);
    Tensor ZH = VH + VH - XH;
    EXPECT_TRUE(allclose(to_host(Z), ZH));
}
#endif
