// TEST INFRASTRUCTURE, not product code. C entry points around the reference's own CPU kernels
// (namespace cpu, src/cpu/*.hpp of the reference), compiled together with the reference's
// sources where they lie into oracle/_ref/libtannic_ref.so. Used to validate the C restatement
// in tannic_oracle.c, to generate the golden fixtures under tests/golden/ and as the
// "reference" CPU baseline of the benchmark.
//
// It also proves, at compile time, that the records of include/tannic_b200.h are
// layout-identical to the reference's runtime PODs.
#include <cstddef>
#include <cstdint>

#include "runtime/resources.h"
#include "runtime/status.h"
#include "runtime/streams.h"
#include "runtime/tensor.h"
#include "runtime/types.h"

#include "cpu/argred.hpp"
#include "cpu/conv.hpp"
#include "cpu/cpy.hpp"
#include "cpu/matmul.hpp"
#include "cpu/ops.hpp"
#include "cpu/val.hpp"
#include "cpu/outer.hpp"
#include "cpu/reps.hpp"
#include "cpu/concat.hpp"
#include "cpu/triang.hpp"
#include "cpu/complex.hpp"
#include "cpu/cmps.hpp"

#include "tannic_b200.h"

using namespace tannic;

static_assert(sizeof(tn_tensor_t) == sizeof(tensor_t), "tensor_t size");
static_assert(offsetof(tn_tensor_t, address) == offsetof(tensor_t, address), "address");
static_assert(offsetof(tn_tensor_t, rank) == offsetof(tensor_t, rank), "rank");
static_assert(offsetof(tn_tensor_t, shape) == offsetof(tensor_t, shape), "shape");
static_assert(offsetof(tn_tensor_t, strides) == offsetof(tensor_t, strides), "strides");
static_assert(offsetof(tn_tensor_t, dtype) == offsetof(tensor_t, dtype), "dtype");
static_assert(offsetof(tn_tensor_t, environment) == offsetof(tensor_t, environment), "environment");
static_assert(offsetof(tn_tensor_t, size) == offsetof(tensor_t, size), "size");
static_assert(offsetof(tn_tensor_t, layout) == offsetof(tensor_t, layout), "layout");
static_assert(sizeof(tn_scalar_t) == sizeof(scalar_t) && offsetof(tn_scalar_t, dtype) == offsetof(scalar_t, dtype), "scalar_t");
static_assert(sizeof(tn_stream_t) == sizeof(stream_t), "stream_t");
static_assert(sizeof(tn_device_t) == sizeof(device_t), "device_t");
static_assert(sizeof(tn_environment_t) == sizeof(environment_t), "environment_t");
static_assert((int)TN_TYPES == (int)TYPES && (int)TN_FLOAT16 == (int)float16 && (int)TN_BFLOAT16 == (int)bfloat16 &&
              (int)TN_FLOAT32 == (int)float32 && (int)TN_FLOAT64 == (int)float64 && (int)TN_INT8 == (int)int8 &&
              (int)TN_INT64 == (int)int64 && (int)TN_COMPLEX128 == (int)complex128, "dtype enum");
static_assert((int)TN_SUCCESS == (int)SUCCESS && (int)TN_ERROR == (int)ERROR && (int)TN_UNSUPPORTED_DTYPE == (int)UNSUPPORTED_DTYPE &&
              (int)TN_NULL_ALLOCATOR == (int)NULL_ALLOCATOR && (int)TN_INCOMPATIBLE_DEVICES == (int)INCOMPATIBLE_DEVICES, "status enum");
static_assert((int)TN_SINGLETON == (int)SINGLETON && (int)TN_CONTIGUOUS == (int)CONTIGUOUS && (int)TN_STRIDED == (int)STRIDED, "layout enum");
static_assert((int)TN_HOST == (int)HOST && (int)TN_DEVICE == (int)DEVICE && (int)TN_PINNED == (int)PINNED, "environment enum");

extern "C" {

int ref_add(const tensor_t* a, const tensor_t* b, tensor_t* d) { return cpu::add(a, b, d); }
int ref_sub(const tensor_t* a, const tensor_t* b, tensor_t* d) { return cpu::sub(a, b, d); }
int ref_mul(const tensor_t* a, const tensor_t* b, tensor_t* d) { return cpu::mul(a, b, d); }
int ref_pow(const tensor_t* a, const tensor_t* b, tensor_t* d) { return cpu::pow(a, b, d); }

int ref_neg(const tensor_t* x, tensor_t* d) { return cpu::neg(x, d); }
int ref_repack(const tensor_t* x, tensor_t* d) { return cpu::repack(x, d); }
int ref_log(const tensor_t* x, tensor_t* d) { return cpu::log(x, d); }
int ref_exp(const tensor_t* x, tensor_t* d) { return cpu::exp(x, d); }
int ref_sqrt(const tensor_t* x, tensor_t* d) { return cpu::sqrt(x, d); }
int ref_rsqrt(const tensor_t* x, tensor_t* d, float eps) { return cpu::rsqrt(x, d, eps); }
int ref_abs(const tensor_t* x, tensor_t* d) { return cpu::abs(x, d); }
int ref_sin(const tensor_t* x, tensor_t* d) { return cpu::sin(x, d); }
int ref_cos(const tensor_t* x, tensor_t* d) { return cpu::cos(x, d); }
int ref_tan(const tensor_t* x, tensor_t* d) { return cpu::tan(x, d); }
int ref_sinh(const tensor_t* x, tensor_t* d) { return cpu::sinh(x, d); }
int ref_cosh(const tensor_t* x, tensor_t* d) { return cpu::cosh(x, d); }
int ref_tanh(const tensor_t* x, tensor_t* d) { return cpu::tanh(x, d); }
int ref_scale(const tensor_t* x, const scalar_t* s, tensor_t* d) { return cpu::scale(x, s, d); }

int ref_gemm(const tensor_t* a, const tensor_t* b, tensor_t* d) { return cpu::gemm(a, b, d); }
int ref_conv2d(const tensor_t* x, const tensor_t* w, tensor_t* y, const size_t pad[2], const size_t stride[2]) {
    return cpu::conv2d(x, w, y, pad, stride);
}
int ref_conv2d_bias(const tensor_t* x, const tensor_t* w, const tensor_t* b, tensor_t* y, const size_t pad[2], const size_t stride[2]) {
    return cpu::conv2d(x, w, b, y, pad, stride);
}

int ref_argmax(const tensor_t* x, tensor_t* d, uint8_t axis) { return cpu::argmax(x, d, axis); }
int ref_argmin(const tensor_t* x, tensor_t* d, uint8_t axis) { return cpu::argmin(x, d, axis); }
int ref_argsum(const tensor_t* x, tensor_t* d, uint8_t axis) { return cpu::argsum(x, d, axis); }
int ref_argmean(const tensor_t* x, tensor_t* d, uint8_t axis) { return cpu::argmean(x, d, axis); }

int ref_cpy(const tensor_t* x, tensor_t* d) { return cpu::cpy(x, d); }
int ref_outer(const tensor_t* a, const tensor_t* b, tensor_t* d) { return cpu::outer(a, b, d); }
int ref_repeat(const tensor_t* x, tensor_t* d, int axis, int reps) { return cpu::repeat(x, d, axis, reps); }
int ref_concat(const tensor_t* a, const tensor_t* b, tensor_t* d, int axis) { return cpu::concat(a, b, d, axis); }
int ref_triu(const tensor_t* x, tensor_t* d, int k) { return cpu::triu(x, d, k); }
int ref_tril(const tensor_t* x, tensor_t* d, int k) { return cpu::tril(x, d, k); }
int ref_view_as_cartesian(const tensor_t* a, const tensor_t* b, tensor_t* d) { return cpu::view_as_cartesian(a, b, d); }
int ref_view_as_polar(const tensor_t* a, const tensor_t* b, tensor_t* d) { return cpu::view_as_polar(a, b, d); }
int ref_conv1d(const tensor_t* x, const tensor_t* w, tensor_t* y, size_t pad, size_t stride) { return cpu::conv1d(x, w, y, pad, stride); }
int ref_eq(const tensor_t* a, const tensor_t* b, tensor_t* d) { return cpu::eq(a, b, d); }
int ref_ne(const tensor_t* a, const tensor_t* b, tensor_t* d) { return cpu::ne(a, b, d); }
int ref_gt(const tensor_t* a, const tensor_t* b, tensor_t* d) { return cpu::gt(a, b, d); }
int ref_ge(const tensor_t* a, const tensor_t* b, tensor_t* d) { return cpu::ge(a, b, d); }
int ref_lt(const tensor_t* a, const tensor_t* b, tensor_t* d) { return cpu::lt(a, b, d); }
int ref_le(const tensor_t* a, const tensor_t* b, tensor_t* d) { return cpu::le(a, b, d); }
int ref_allclose(const tensor_t* a, const tensor_t* b, double rtol, double atol) {
    try {
        return cpu::allclose(a, b, rtol, atol) ? 1 : 0;
    } catch (...) {
        return -1;
    }
}

}  // extern "C"
