// Shared host/device helpers for the sm_100a backend: status + error text, dtype traits,
// runtime-typed loads/stores for the generic paths, launch accounting.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>

#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "tannic_b200.h"
#include "numeric.cuh"

namespace tnb {

// ---------------------------------------------------------------- errors -------------
// The reference's device helpers print and exit() on a CUDA error (src/cuda/exc.cuh:8-16);
// here every failure becomes a status plus a per-thread message.
char* error_buffer();  // thread-local, 512 bytes
tn_status fail(tn_status code, const char* fmt, ...);

#define TN_CUDA(call)                                                                      \
    do {                                                                                   \
        cudaError_t err__ = (call);                                                        \
        if (err__ != cudaSuccess)                                                          \
            return ::tnb::fail(TN_ERROR, "%s failed: %s (%s:%d)", #call,                   \
                               cudaGetErrorString(err__), __FILE__, __LINE__);             \
    } while (0)

#define TN_TRY(expr)                                  \
    do {                                              \
        tn_status st__ = (expr);                      \
        if (st__ != TN_SUCCESS) return st__;          \
    } while (0)

extern std::atomic<uint64_t> g_launches;
inline void count_launch(uint64_t n = 1) { g_launches.fetch_add(n, std::memory_order_relaxed); }

// Checks the launch that was just issued (pattern of src/cuda/argred.cu:138) and counts it.
tn_status after_launch(const char* what);

inline cudaStream_t as_cuda(tn_stream_t s) { return reinterpret_cast<cudaStream_t>(s.address); }

// Makes the device that owns `t` current for this thread (cheap when unchanged). Device entry
// points refuse host tensors: there is no CPU fallback on this path.
tn_status use_device_of(const tn_tensor_t* t);
tn_status use_device(int id);

// ---------------------------------------------------------------- dtypes -------------
__host__ __device__ inline int dtype_bytes(int dt) {
    switch (dt) {
        case TN_BOOLEAN: case TN_INT8: return 1;
        case TN_INT16: case TN_FLOAT16: case TN_BFLOAT16: return 2;
        case TN_INT32: case TN_FLOAT32: return 4;
        case TN_INT64: case TN_FLOAT64: case TN_COMPLEX64: return 8;
        case TN_COMPLEX128: return 16;
        default: return 0;
    }
}
inline bool is_int(int dt) { return dt >= TN_INT8 && dt <= TN_INT64; }
inline bool is_half(int dt) { return dt == TN_FLOAT16 || dt == TN_BFLOAT16; }
inline bool is_float(int dt) { return dt >= TN_FLOAT16 && dt <= TN_FLOAT64; }
inline bool is_numeric(int dt) { return dt >= TN_INT8 && dt <= TN_FLOAT64; }

template <typename T> struct dtype_of;
template <> struct dtype_of<int8_t> { static constexpr int value = TN_INT8; };
template <> struct dtype_of<int16_t> { static constexpr int value = TN_INT16; };
template <> struct dtype_of<int32_t> { static constexpr int value = TN_INT32; };
template <> struct dtype_of<int64_t> { static constexpr int value = TN_INT64; };
template <> struct dtype_of<__half> { static constexpr int value = TN_FLOAT16; };
template <> struct dtype_of<__nv_bfloat16> { static constexpr int value = TN_BFLOAT16; };
template <> struct dtype_of<float> { static constexpr int value = TN_FLOAT32; };
template <> struct dtype_of<double> { static constexpr int value = TN_FLOAT64; };

// Runtime-typed element access for the generic (any dtype pair, any strides) kernels.
// C is float, double or int64_t. Integer sources feeding a float32 class convert int -> float
// directly (as the C++ expression `int32_t + float` does).
template <typename C>
__device__ __forceinline__ C load_as(const void* base, int dt, int64_t idx) {
    switch (dt) {
        case TN_INT8: return static_cast<C>(static_cast<const int8_t*>(base)[idx]);
        case TN_INT16: return static_cast<C>(static_cast<const int16_t*>(base)[idx]);
        case TN_INT32: return static_cast<C>(static_cast<const int32_t*>(base)[idx]);
        case TN_INT64: return static_cast<C>(static_cast<const int64_t*>(base)[idx]);
        case TN_FLOAT16: return static_cast<C>(__half2float(static_cast<const __half*>(base)[idx]));
        case TN_BFLOAT16: return static_cast<C>(__bfloat162float(static_cast<const __nv_bfloat16*>(base)[idx]));
        case TN_FLOAT32: return static_cast<C>(static_cast<const float*>(base)[idx]);
        case TN_FLOAT64: return static_cast<C>(static_cast<const double*>(base)[idx]);
        default: return C(0);
    }
}

template <typename C>
__device__ __forceinline__ void store_as(void* base, int dt, int64_t idx, C v) {
    switch (dt) {
        case TN_INT8: static_cast<int8_t*>(base)[idx] = static_cast<int8_t>(static_cast<int64_t>(v)); break;
        case TN_INT16: static_cast<int16_t*>(base)[idx] = static_cast<int16_t>(static_cast<int64_t>(v)); break;
        case TN_INT32: static_cast<int32_t*>(base)[idx] = static_cast<int32_t>(static_cast<int64_t>(v)); break;
        case TN_INT64: static_cast<int64_t*>(base)[idx] = static_cast<int64_t>(v); break;
        case TN_FLOAT16: static_cast<__half*>(base)[idx] = from_compute<__half, C>(v); break;
        case TN_BFLOAT16: static_cast<__nv_bfloat16*>(base)[idx] = from_compute<__nv_bfloat16, C>(v); break;
        case TN_FLOAT32: static_cast<float*>(base)[idx] = static_cast<float>(v); break;
        case TN_FLOAT64: static_cast<double*>(base)[idx] = static_cast<double>(v); break;
        default: break;
    }
}

// Tuning knobs from the environment (launch geometry only; results never depend on them). Each
// name is looked up once per process; later calls return the remembered value. `name` must be a
// string literal (the cache is keyed by its address). Values <= 0 or unset give `fallback`.
int env_knob(const char* name, int fallback);

// ---------------------------------------------------------------- geometry -----------
// Number of SMs of the current device (148 on B200); grids of the streaming kernels are sized
// as a multiple of it.
int sm_count();
int sm_margin();  // SMs the persistent GEMM kernels leave to kernels of other streams (0 by default)

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Stream-ordered scratch from the device's pool (cudaMallocAsync on `stream`); freed with
// scratch_free on the same stream after the consuming kernel has been enqueued.
tn_status scratch_alloc(void** ptr, size_t nbytes, cudaStream_t stream);
tn_status scratch_free(void* ptr, cudaStream_t stream);

// Called by the entry points that synchronise with the device (tn_stream_synchronize,
// tn_copy_to_host, tn_allclose) after the device is idle: if a CTA gave up on a bounded wait since
// the last such call on the current device, the results it owed were never written, so the call
// reports TN_ERROR with a message instead of SUCCESS.
tn_status surface_device_aborts();

}  // namespace tnb
