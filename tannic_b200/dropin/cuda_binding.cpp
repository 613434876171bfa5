// Drop-in binding: defines every `cuda::` symbol that the reference's host translation units
// reference under -DCUDA (src/operations.cpp, functions.cpp, transformations.cpp, convolutions.cpp,
// reductions.cpp, resources.cpp, bindings.cpp, tensor.cpp, comparisons.cpp, IO.cpp, filter.cpp,
// complex.cpp) by forwarding to the C ABI of libtannic_b200.so. It is compiled against the
// reference's own headers (their declarations are the contract), replaces all of src/cuda/*.cu and
// needs no other change to the reference.
#include <cstdint>
#include <new>
#include <stdexcept>

#include "cuda/argred.cuh"
#include "cuda/complex.cuh"
#include "cuda/concat.cuh"
#include "cuda/conv.cuh"
#include "cuda/cpy.cuh"
#include "cuda/matmul.cuh"
#include "cuda/mem.cuh"
#include "cuda/ops.cuh"
#include "cuda/outer.cuh"
#include "cuda/reps.cuh"
#include "cuda/streams.cuh"
#include "cuda/triang.cuh"
#include "cuda/val.cuh"

#include "tannic_b200.h"

namespace {
inline const tn_tensor_t* in(const tensor_t* t) { return reinterpret_cast<const tn_tensor_t*>(t); }
inline tn_tensor_t* out(tensor_t* t) { return reinterpret_cast<tn_tensor_t*>(t); }
inline tn_stream_t on(stream_t s) { return tn_stream_t{s.address}; }
inline status st(tn_status s) { return static_cast<status>(s); }
inline const tn_device_t* dev(const device_t* d) { return reinterpret_cast<const tn_device_t*>(d); }
}  // namespace

namespace cuda {

status add(const tensor_t* a, const tensor_t* b, tensor_t* d, stream_t s) { return st(tn_add(in(a), in(b), out(d), on(s))); }
status sub(const tensor_t* a, const tensor_t* b, tensor_t* d, stream_t s) { return st(tn_sub(in(a), in(b), out(d), on(s))); }
status mul(const tensor_t* a, const tensor_t* b, tensor_t* d, stream_t s) { return st(tn_mul(in(a), in(b), out(d), on(s))); }
status pow(const tensor_t* a, const tensor_t* b, tensor_t* d, stream_t s) { return st(tn_pow(in(a), in(b), out(d), on(s))); }
status scale(const tensor_t* x, const scalar_t* k, tensor_t* d, stream_t s) {
    return st(tn_scale(in(x), reinterpret_cast<const tn_scalar_t*>(k), out(d), on(s)));
}

status neg(const tensor_t* x, tensor_t* d, stream_t s) { return st(tn_neg(in(x), out(d), on(s))); }
status repack(const tensor_t* x, tensor_t* d, stream_t s) { return st(tn_repack(in(x), out(d), on(s))); }
status log(const tensor_t* x, tensor_t* d, stream_t s) { return st(tn_log(in(x), out(d), on(s))); }
status exp(const tensor_t* x, tensor_t* d, stream_t s) { return st(tn_exp(in(x), out(d), on(s))); }
status sqrt(const tensor_t* x, tensor_t* d, stream_t s) { return st(tn_sqrt(in(x), out(d), on(s))); }
status rsqrt(const tensor_t* x, tensor_t* d, stream_t s, float eps) { return st(tn_rsqrt(in(x), out(d), on(s), eps)); }
status abs(const tensor_t* x, tensor_t* d, stream_t s) { return st(tn_abs(in(x), out(d), on(s))); }
status sin(const tensor_t* x, tensor_t* d, stream_t s) { return st(tn_sin(in(x), out(d), on(s))); }
status cos(const tensor_t* x, tensor_t* d, stream_t s) { return st(tn_cos(in(x), out(d), on(s))); }
status tan(const tensor_t* x, tensor_t* d, stream_t s) { return st(tn_tan(in(x), out(d), on(s))); }
status sinh(const tensor_t* x, tensor_t* d, stream_t s) { return st(tn_sinh(in(x), out(d), on(s))); }
status cosh(const tensor_t* x, tensor_t* d, stream_t s) { return st(tn_cosh(in(x), out(d), on(s))); }
status tanh(const tensor_t* x, tensor_t* d, stream_t s) { return st(tn_tanh(in(x), out(d), on(s))); }

status gemm(const tensor_t* a, const tensor_t* b, tensor_t* d, stream_t s) { return st(tn_gemm(in(a), in(b), out(d), on(s))); }

status conv2d(const tensor_t* x, const tensor_t* w, tensor_t* y, stream_t s, const size_t pad[2], const size_t stride[2]) {
    return st(tn_conv2d(in(x), in(w), out(y), on(s), pad, stride));
}
status conv2d(const tensor_t* x, const tensor_t* w, const tensor_t* b, tensor_t* y, stream_t s, const size_t pad[2],
              const size_t stride[2]) {
    return st(tn_conv2d_bias(in(x), in(w), in(b), out(y), on(s), pad, stride));
}

status conv1d(const tensor_t* x, const tensor_t* w, tensor_t* y, stream_t s, const size_t pad, const size_t stride) {
    return st(tn_conv1d(in(x), in(w), out(y), on(s), pad, stride));
}

status argmax(const tensor_t* x, tensor_t* d, stream_t s, uint8_t ax) { return st(tn_argmax(in(x), out(d), on(s), ax)); }
status argmin(const tensor_t* x, tensor_t* d, stream_t s, uint8_t ax) { return st(tn_argmin(in(x), out(d), on(s), ax)); }
status argsum(const tensor_t* x, tensor_t* d, stream_t s, uint8_t ax) { return st(tn_argsum(in(x), out(d), on(s), ax)); }
status argmean(const tensor_t* x, tensor_t* d, stream_t s, uint8_t ax) { return st(tn_argmean(in(x), out(d), on(s), ax)); }

status cpy(const tensor_t* x, tensor_t* d, stream_t s) { return st(tn_cpy(in(x), out(d), on(s))); }
bool allclose(const tensor_t* a, const tensor_t* b, stream_t s, double rtol, double atol) {
    int close = 0;
    if (tn_allclose(in(a), in(b), on(s), rtol, atol, &close) != TN_SUCCESS) throw std::runtime_error(tn_last_error());
    return close != 0;
}

// ---- data movement around the operator hot path ---------------------------------------------------
status outer(tensor_t const* a, tensor_t const* b, tensor_t* d, stream_t s) { return st(tn_outer(in(a), in(b), out(d), on(s))); }
status repeat(const tensor_t* x, tensor_t* d, int axis, int reps, stream_t s) { return st(tn_repeat(in(x), out(d), axis, reps, on(s))); }
status concat(const tensor_t* a, const tensor_t* b, tensor_t* d, stream_t s, int axis) { return st(tn_concat(in(a), in(b), out(d), on(s), axis)); }
status triu(const tensor_t* x, tensor_t* d, stream_t s, int k) { return st(tn_triu(in(x), out(d), on(s), k)); }
status tril(const tensor_t* x, tensor_t* d, stream_t s, int k) { return st(tn_tril(in(x), out(d), on(s), k)); }
status view_as_cartesian(tensor_t const* re, tensor_t const* im, tensor_t* d, stream_t s) { return st(tn_view_as_cartesian(in(re), in(im), out(d), on(s))); }
status view_as_polar(const tensor_t* rho, const tensor_t* theta, tensor_t* d, stream_t s) { return st(tn_view_as_polar(in(rho), in(theta), out(d), on(s))); }

// ---- memory and streams --------------------------------------------------------------------------
int getDeviceCount() {
    int n = 0;
    tn_device_count(&n);
    return n;
}
void setDevice(int id) { tn_set_device(id); }
void* allocate(const device_t* d, size_t nbytes) {
    void* p = nullptr;
    if (tn_allocate(dev(d), nbytes, &p) != TN_SUCCESS) throw std::bad_alloc();
    return p;
}
void* deallocate(const device_t* d, void* p) {
    tn_deallocate(dev(d), p);
    return nullptr;
}
void copyFromHost(const device_t* d, const void* h, void* p, size_t n) {
    // element-sized writes are Tensor::assign filling a tensor from an initializer list (src/tensor.cpp:34-44):
    // they are gathered into one copy per contiguous run
    const tn_status rc = n <= 16 ? tn_assign_from_host(dev(d), h, p, n) : tn_copy_from_host(dev(d), h, p, n);
    if (rc != TN_SUCCESS) throw std::runtime_error(tn_last_error());
}
void copyDeviceToHost(const device_t* d, const void* p, void* h, size_t n) {
    if (tn_copy_to_host(dev(d), p, h, n) != TN_SUCCESS) throw std::runtime_error(tn_last_error());
}
bool compareFromHost(const device_t* d, const void* h, const void* p, size_t n) {
    int eq = 0;
    if (tn_compare_from_host(dev(d), h, p, n, &eq) != TN_SUCCESS) throw std::runtime_error(tn_last_error());
    return eq != 0;
}
status copy(const tensor_t* src, tensor_t* dst, size_t nbytes, stream_t s) { return st(tn_copy(in(src), out(dst), nbytes, on(s))); }

// The stream pool behind tannic::pop_stream / put_stream (src/bindings.cpp:22-42) lives in the backend.
Streams::Streams() {}
Streams::~Streams() {}
cudaStream_t Streams::pop(int device) {
    tn_device_t d{device};
    tn_stream_t s{0};
    if (tn_stream_pop(&d, &s) != TN_SUCCESS) throw std::runtime_error(tn_last_error());
    return reinterpret_cast<cudaStream_t>(s.address);
}
void Streams::put(int device, cudaStream_t stream) {
    tn_device_t d{device};
    tn_stream_put(&d, tn_stream_t{reinterpret_cast<uintptr_t>(stream)});
}

}  // namespace cuda
