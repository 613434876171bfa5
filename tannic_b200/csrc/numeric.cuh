// Storage type <-> arithmetic type conversions shared by every kernel. This header is also
// handed, as text, to the run-time compiler that instantiates fused element-wise programs, so it
// names nothing from the host's standard library.
#pragma once

#include <cuda_fp16.h>
#include <cuda_bf16.h>

#ifdef __CUDACC_RTC__
#include <cuda/std/cstdint>
#include <cuda/std/type_traits>
namespace tnb { namespace stdx = ::cuda::std; }
using ::cuda::std::int8_t;
using ::cuda::std::int16_t;
using ::cuda::std::int32_t;
using ::cuda::std::int64_t;
using ::cuda::std::uint8_t;
using ::cuda::std::uint16_t;
using ::cuda::std::uint32_t;
using ::cuda::std::uint64_t;
#else
#include <cstdint>
#include <type_traits>
namespace tnb { namespace stdx = ::std; }
#endif

namespace tnb {

// Arithmetic type a storage type computes in: half types in float32 (rounded once on store,
// as src/cuda/ops-unary.cu:116-136 does), integers in their own width (wrapping).
template <typename T> struct compute_of { using type = T; };
template <> struct compute_of<__half> { using type = float; };
template <> struct compute_of<__nv_bfloat16> { using type = float; };

template <typename C, typename T> __device__ __forceinline__ C to_compute(T v) { return static_cast<C>(v); }
template <> __device__ __forceinline__ float to_compute<float, __half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_compute<float, __nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ double to_compute<double, __half>(__half v) { return (double)__half2float(v); }
template <> __device__ __forceinline__ double to_compute<double, __nv_bfloat16>(__nv_bfloat16 v) { return (double)__bfloat162float(v); }

template <typename T, typename C> __device__ __forceinline__ T from_compute(C v) { return static_cast<T>(v); }
template <> __device__ __forceinline__ __half from_compute<__half, float>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_compute<__nv_bfloat16, float>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_compute<__half, double>(double v) { return __double2half(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_compute<__nv_bfloat16, double>(double v) { return __double2bfloat16(v); }

template <> __device__ __forceinline__ __half from_compute<__half, int64_t>(int64_t v) { return __float2half_rn((float)v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_compute<__nv_bfloat16, int64_t>(int64_t v) { return __float2bfloat16_rn((float)v); }

}  // namespace tnb
