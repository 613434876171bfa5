// Strided copy (slice assignment) and tolerance comparison. Replace src/cuda/cpy.cu and
// src/cuda/val.cu of the reference.
#include "common.cuh"

namespace tnb {
namespace {

constexpr int kThreads = 256;

struct PairGeom {
    int rank;
    int64_t n;
    int64_t sizes[TN_MAX_RANK];
    int64_t sa[TN_MAX_RANK];
    int64_t sb[TN_MAX_RANK];
};

__device__ __forceinline__ void decode(const PairGeom& g, int64_t lin, int64_t& oa, int64_t& ob) {
    oa = ob = 0;
    for (int d = g.rank - 1; d >= 0; --d) {
        const int64_t c = lin % g.sizes[d];
        lin /= g.sizes[d];
        oa += c * g.sa[d];
        ob += c * g.sb[d];
    }
}

// dst[off_b(i)] = src[off_a(i)] for every logical index i, moving elements as raw words.
template <typename W>
__global__ void __launch_bounds__(kThreads) cpy_strided(const W* __restrict__ src, W* __restrict__ dst, PairGeom g) {
    const int64_t step = (int64_t)gridDim.x * kThreads;
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < g.n; i += step) {
        int64_t oa, ob;
        decode(g, i, oa, ob);
        dst[ob] = src[oa];
    }
}

// Tiled transpose for views whose unit-stride dimension is not the result's: 32 x 32 element tiles
// through shared memory, read along the source's unit-stride dimension `jd`, written along the
// result's last one. The other dimensions are decoded once per tile.
template <typename W>
__global__ void __launch_bounds__(kThreads) cpy_transposed(const W* __restrict__ src, W* __restrict__ dst, PairGeom g, int jd,
                                                           int64_t tiles_j, int64_t tiles_l, int64_t tiles) {
    __shared__ W tile[32][33];
    const int last = g.rank - 1;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
    const int64_t J = g.sizes[jd], L = g.sizes[last];
    for (int64_t t = blockIdx.x; t < tiles; t += gridDim.x) {
        const int64_t tl = t % tiles_l;
        int64_t rest = t / tiles_l;
        const int64_t tj = rest % tiles_j;
        rest /= tiles_j;
        int64_t oa = 0, ob = 0;
        for (int d = last - 1; d >= 0; --d) {
            if (d == jd) continue;
            const int64_t c = rest % g.sizes[d];
            rest /= g.sizes[d];
            oa += c * g.sa[d];
            ob += c * g.sb[d];
        }
        const int64_t j0 = tj * 32, l0 = tl * 32;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int64_t l = l0 + ty + 8 * i, j = j0 + tx;
            if (l < L && j < J) tile[ty + 8 * i][tx] = src[oa + j * g.sa[jd] + l * g.sa[last]];
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int64_t j = j0 + ty + 8 * i, l = l0 + tx;
            if (j < J && l < L) dst[ob + j * g.sb[jd] + l * g.sb[last]] = tile[tx][ty + 8 * i];
        }
        __syncthreads();
    }
}

// The same for 2-byte elements, two at a time: 64 x 64 tiles, 4-byte global loads along the
// source's unit-stride dimension and 4-byte global stores along the result's (128 bytes per warp
// row either way). Needs even extents, even strides and 4-byte aligned bases (checked on the host).
__global__ void __launch_bounds__(kThreads) cpy_transposed_pairs(const uint16_t* __restrict__ src, uint16_t* __restrict__ dst, PairGeom g,
                                                                 int jd, int64_t tiles_j, int64_t tiles_l, int64_t tiles) {
    __shared__ uint16_t tile[64][66];  // [l][j], 33-word pitch
    const int last = g.rank - 1;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 lanes x 8 rows per pass
    const int64_t J = g.sizes[jd], L = g.sizes[last];
    for (int64_t t = blockIdx.x; t < tiles; t += gridDim.x) {
        const int64_t tl = t % tiles_l;
        int64_t rest = t / tiles_l;
        const int64_t tj = rest % tiles_j;
        rest /= tiles_j;
        int64_t oa = 0, ob = 0;
        for (int d = last - 1; d >= 0; --d) {
            if (d == jd) continue;
            const int64_t c = rest % g.sizes[d];
            rest /= g.sizes[d];
            oa += c * g.sa[d];
            ob += c * g.sb[d];
        }
        const int64_t j0 = tj * 64, l0 = tl * 64;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int64_t l = l0 + ty + 8 * i, j = j0 + 2 * tx;
            if (l < L && j < J)  // J is even: the pair is inside or outside as a whole
                *reinterpret_cast<uint32_t*>(&tile[ty + 8 * i][2 * tx]) = *reinterpret_cast<const uint32_t*>(src + oa + j + l * g.sa[last]);
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int64_t j = j0 + ty + 8 * i, l = l0 + 2 * tx;
            if (j < J && l < L) {
                const uint32_t pair = static_cast<uint32_t>(tile[2 * tx][ty + 8 * i]) | (static_cast<uint32_t>(tile[2 * tx + 1][ty + 8 * i]) << 16);
                *reinterpret_cast<uint32_t*>(dst + ob + j * g.sb[jd] + l) = pair;
            }
        }
        __syncthreads();
    }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) allclose_kernel(const T* __restrict__ a, const T* __restrict__ b, PairGeom g,
                                                            double rtol, double atol, int* mismatch) {
    const int64_t step = (int64_t)gridDim.x * kThreads;
    bool bad = false;
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < g.n; i += step) {
        int64_t oa, ob;
        decode(g, i, oa, ob);
        const double x = to_compute<double>(a[oa]), y = to_compute<double>(b[ob]);
        // a NaN on either side never trips this test, exactly as in src/cuda/val.cu:8-40
        if (fabs(x - y) > atol + rtol * fabs(y)) bad = true;
    }
    if (__syncthreads_or(bad) && threadIdx.x == 0) atomicOr(mismatch, 1);
}

// Elementwise comparison into a bit-packed boolean result: element i of the result (logical row-major
// order) is bit i % 8 of byte i / 8, the layout the reference's CPU kernel writes
// (src/cpu/cmps.cpp:16-41) and its boolean tensors use (nbytesof, include/tannic/types.hpp:149-154).
// A thread produces one byte from eight consecutive elements, so no two threads touch one byte and
// the padding bits of the last byte are written as zero. IEEE semantics: every comparison with a NaN
// is false except !=.
enum { CMP_EQ = 0, CMP_NE, CMP_GT, CMP_GE, CMP_LT, CMP_LE };
template <int OP, typename C> __device__ __forceinline__ bool compare(C x, C y) {
    if constexpr (OP == CMP_EQ) return x == y;
    else if constexpr (OP == CMP_NE) return x != y;
    else if constexpr (OP == CMP_GT) return x > y;
    else if constexpr (OP == CMP_GE) return x >= y;
    else if constexpr (OP == CMP_LT) return x < y;
    else return x <= y;
}
template <typename T, int OP>
__global__ void __launch_bounds__(kThreads) compare_bits(const T* __restrict__ a, const T* __restrict__ b, uint8_t* __restrict__ dst, PairGeom g,
                                                         int dense) {
    using C = typename compute_of<T>::type;  // 16-bit floats compare as float32 (exact)
    const int64_t nbytes = (g.n + 7) >> 3;
    const int64_t step = (int64_t)gridDim.x * kThreads;
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < nbytes; i += step) {
        const int64_t first = i * 8;
        unsigned bits = 0;
        if (dense && first + 8 <= g.n) {
#pragma unroll
            for (int k = 0; k < 8; ++k) bits |= (compare<OP, C>(to_compute<C>(a[first + k]), to_compute<C>(b[first + k])) ? 1u : 0u) << k;
        } else {
            for (int k = 0; k < 8 && first + k < g.n; ++k) {
                int64_t oa, ob;
                decode(g, first + k, oa, ob);
                bits |= (compare<OP, C>(to_compute<C>(a[oa]), to_compute<C>(b[ob])) ? 1u : 0u) << k;
            }
        }
        dst[i] = static_cast<uint8_t>(bits);
    }
}

// Geometry over `shape_of`'s logical shape; extent-1 dims of either side read offset 0
// (src/cpu/cpy.cpp:19-43).
void make_geom(const tn_tensor_t* a, const tn_tensor_t* b, const tn_tensor_t* shape_of, PairGeom& g) {
    int64_t sizes[TN_MAX_RANK], sa[TN_MAX_RANK], sb[TN_MAX_RANK];
    int rank = 0;
    g.n = 1;
    for (int d = 0; d < shape_of->rank; ++d) {
        const int64_t sz = (int64_t)shape_of->shape.sizes[d];
        g.n *= sz;
        if (sz == 1) continue;  // contributes offset 0 on both sides
        sizes[rank] = sz;
        sa[rank] = a->shape.sizes[d] == 1 ? 0 : a->strides.sizes[d];
        sb[rank] = b->shape.sizes[d] == 1 ? 0 : b->strides.sizes[d];
        ++rank;
    }
    // merge neighbours that both sides walk as one run: fewer divisions per element
    g.rank = 0;
    for (int d = 0; d < rank; ++d) {
        if (g.rank > 0 && g.sa[g.rank - 1] == sa[d] * sizes[d] && g.sb[g.rank - 1] == sb[d] * sizes[d]) {
            g.sizes[g.rank - 1] *= sizes[d];
            g.sa[g.rank - 1] = sa[d];
            g.sb[g.rank - 1] = sb[d];
        } else {
            g.sizes[g.rank] = sizes[d];
            g.sa[g.rank] = sa[d];
            g.sb[g.rank] = sb[d];
            ++g.rank;
        }
    }
}

int grid_for(int64_t n) {
    const int64_t cap = (int64_t)sm_count() * 8;
    int64_t blocks = ceil_div(n, kThreads);
    if (blocks < 1) blocks = 1;
    return (int)(blocks < cap ? blocks : cap);
}

}  // namespace
}  // namespace tnb

using namespace tnb;

namespace {
template <int OP>
tn_status compare_entry(const tn_tensor_t* a, const tn_tensor_t* b, tn_tensor_t* dst, tn_stream_t stream) {
    if (!a || !b || !dst) return fail(TN_ERROR, "null tensor");
    if (a->dtype != b->dtype || !is_numeric(a->dtype)) return fail(TN_UNSUPPORTED_DTYPE, "comparison: dtypes %d and %d", (int)a->dtype, (int)b->dtype);
    if (dst->dtype != TN_BOOLEAN) return fail(TN_UNSUPPORTED_DTYPE, "comparison: the result must be boolean, got %d", (int)dst->dtype);
    if (a->rank != dst->rank || b->rank != dst->rank) return fail(TN_ERROR, "comparison: ranks %d, %d -> %d differ", (int)a->rank, (int)b->rank, (int)dst->rank);
    for (int d = 0; d < dst->rank; ++d) {
        const size_t n = dst->shape.sizes[d];
        if ((a->shape.sizes[d] != n && a->shape.sizes[d] != 1) || (b->shape.sizes[d] != n && b->shape.sizes[d] != 1))
            return fail(TN_ERROR, "comparison: operand shapes do not match the result in dimension %d", d);
    }
    if (a->environment.kind != TN_DEVICE || b->environment.kind != TN_DEVICE || dst->environment.kind != TN_DEVICE ||
        a->environment.resource.device.id != b->environment.resource.device.id ||
        a->environment.resource.device.id != dst->environment.resource.device.id)
        return fail(TN_INCOMPATIBLE_DEVICES, "operands must live on one device");
    TN_TRY(use_device_of(dst));
    PairGeom g;
    make_geom(a, b, dst, g);
    if (g.n == 0) return TN_SUCCESS;
    const int dense = g.rank == 0 || (g.rank == 1 && g.sa[0] == 1 && g.sb[0] == 1);
    cudaStream_t s = as_cuda(stream);
    const int grid = grid_for((g.n + 7) / 8);
    uint8_t* out = static_cast<uint8_t*>(dst->address);
#define TN_CMP(T) compare_bits<T, OP><<<grid, kThreads, 0, s>>>(static_cast<const T*>(a->address), static_cast<const T*>(b->address), out, g, dense)
    switch (a->dtype) {
        case TN_INT8: TN_CMP(int8_t); break;
        case TN_INT16: TN_CMP(int16_t); break;
        case TN_INT32: TN_CMP(int32_t); break;
        case TN_INT64: TN_CMP(int64_t); break;
        case TN_FLOAT16: TN_CMP(__half); break;
        case TN_BFLOAT16: TN_CMP(__nv_bfloat16); break;
        case TN_FLOAT32: TN_CMP(float); break;
        default: TN_CMP(double); break;
    }
#undef TN_CMP
    return after_launch("compare_bits");
}
}  // namespace

extern "C" {

tn_status tn_cpy(const tn_tensor_t* src, tn_tensor_t* dst, tn_stream_t stream) {
    if (!src || !dst) return fail(TN_ERROR, "null tensor");
    if (src->dtype != dst->dtype || dtype_bytes(src->dtype) == 0)
        return fail(TN_UNSUPPORTED_DTYPE, "cpy: dtypes %d -> %d", (int)src->dtype, (int)dst->dtype);
    if (src->rank != dst->rank) return fail(TN_ERROR, "cpy: ranks %d and %d differ", (int)src->rank, (int)dst->rank);
    if (src->environment.kind != TN_DEVICE || dst->environment.kind != TN_DEVICE ||
        src->environment.resource.device.id != dst->environment.resource.device.id)
        return fail(TN_INCOMPATIBLE_DEVICES, "operands must live on one device");
    TN_TRY(use_device_of(dst));
    PairGeom g;
    make_geom(src, dst, dst, g);
    if (g.n == 0) return TN_SUCCESS;
    cudaStream_t s = as_cuda(stream);
    // Runs that are contiguous on both sides move as 16-byte words when everything lines up:
    // the innermost extent, every other stride and both base addresses in units of 16 bytes.
    {
        const int64_t esize = dtype_bytes(src->dtype);
        const int64_t pack = 16 / esize;
        const int last = g.rank - 1;
        bool wide = esize < 16 && last >= 0 && g.sa[last] == 1 && g.sb[last] == 1 && g.sizes[last] % pack == 0 &&
                    (reinterpret_cast<uintptr_t>(src->address) & 15) == 0 && (reinterpret_cast<uintptr_t>(dst->address) & 15) == 0;
        for (int d = 0; wide && d < last; ++d) wide = g.sa[d] % pack == 0 && g.sb[d] % pack == 0;
        if (wide) {
            PairGeom w = g;
            w.sizes[last] /= pack;
            w.n /= pack;
            for (int d = 0; d < last; ++d) {
                w.sa[d] /= pack;
                w.sb[d] /= pack;
            }
            cpy_strided<uint4><<<grid_for(w.n), kThreads, 0, s>>>(static_cast<const uint4*>(src->address), static_cast<uint4*>(dst->address), w);
            return after_launch("cpy_strided");
        }
    }
    // A transposing view: the source is contiguous along a dimension that is not the result's last.
    {
        const int last = g.rank - 1;
        int jd = -1;
        if (last >= 1 && g.sb[last] == 1 && g.sa[last] != 1 && g.sizes[last] >= 16)
            for (int d = 0; d < last; ++d)
                if (g.sa[d] == 1 && g.sizes[d] >= 16) jd = d;
        const int esize = dtype_bytes(src->dtype);
        if (jd >= 0 && esize <= 8) {
            int64_t outer = 1;
            for (int d = 0; d < last; ++d)
                if (d != jd) outer *= g.sizes[d];
            const int64_t cap = (int64_t)sm_count() * 16;
            if (esize == 2) {
                bool pairs = g.sizes[jd] % 2 == 0 && g.sizes[last] % 2 == 0 && (reinterpret_cast<uintptr_t>(src->address) & 3) == 0 &&
                             (reinterpret_cast<uintptr_t>(dst->address) & 3) == 0;
                for (int d = 0; pairs && d <= last; ++d) {
                    if (d != jd && g.sa[d] % 2 != 0) pairs = false;
                    if (d != last && g.sb[d] % 2 != 0) pairs = false;
                }
                if (pairs) {
                    const int64_t tj = ceil_div(g.sizes[jd], 64), tl = ceil_div(g.sizes[last], 64), n_tiles = outer * tj * tl;
                    cpy_transposed_pairs<<<(int)(n_tiles < cap ? n_tiles : cap), kThreads, 0, s>>>(
                        static_cast<const uint16_t*>(src->address), static_cast<uint16_t*>(dst->address), g, jd, tj, tl, n_tiles);
                    return after_launch("cpy_transposed_pairs");
                }
            }
            const int64_t tiles_j = ceil_div(g.sizes[jd], 32), tiles_l = ceil_div(g.sizes[last], 32);
            const int64_t tiles = outer * tiles_j * tiles_l;
            const int tgrid = (int)(tiles < cap ? tiles : cap);
            switch (esize) {
                case 1: cpy_transposed<uint8_t><<<tgrid, kThreads, 0, s>>>(static_cast<const uint8_t*>(src->address), static_cast<uint8_t*>(dst->address), g, jd, tiles_j, tiles_l, tiles); break;
                case 2: cpy_transposed<uint16_t><<<tgrid, kThreads, 0, s>>>(static_cast<const uint16_t*>(src->address), static_cast<uint16_t*>(dst->address), g, jd, tiles_j, tiles_l, tiles); break;
                case 4: cpy_transposed<uint32_t><<<tgrid, kThreads, 0, s>>>(static_cast<const uint32_t*>(src->address), static_cast<uint32_t*>(dst->address), g, jd, tiles_j, tiles_l, tiles); break;
                default: cpy_transposed<uint64_t><<<tgrid, kThreads, 0, s>>>(static_cast<const uint64_t*>(src->address), static_cast<uint64_t*>(dst->address), g, jd, tiles_j, tiles_l, tiles); break;
            }
            return after_launch("cpy_transposed");
        }
    }
    const int grid = grid_for(g.n);
    switch (dtype_bytes(src->dtype)) {
        case 1: cpy_strided<uint8_t><<<grid, kThreads, 0, s>>>(static_cast<const uint8_t*>(src->address), static_cast<uint8_t*>(dst->address), g); break;
        case 2: cpy_strided<uint16_t><<<grid, kThreads, 0, s>>>(static_cast<const uint16_t*>(src->address), static_cast<uint16_t*>(dst->address), g); break;
        case 4: cpy_strided<uint32_t><<<grid, kThreads, 0, s>>>(static_cast<const uint32_t*>(src->address), static_cast<uint32_t*>(dst->address), g); break;
        case 8: cpy_strided<uint64_t><<<grid, kThreads, 0, s>>>(static_cast<const uint64_t*>(src->address), static_cast<uint64_t*>(dst->address), g); break;
        default: cpy_strided<uint4><<<grid, kThreads, 0, s>>>(static_cast<const uint4*>(src->address), static_cast<uint4*>(dst->address), g); break;
    }
    return after_launch("cpy_strided");
}

tn_status tn_allclose(const tn_tensor_t* a, const tn_tensor_t* b, tn_stream_t stream, double rtol, double atol, int* close) {
    if (!a || !b || !close) return fail(TN_ERROR, "null argument");
    if (a->dtype != b->dtype || !is_float(a->dtype))
        return fail(TN_UNSUPPORTED_DTYPE, "allclose: dtypes %d and %d", (int)a->dtype, (int)b->dtype);
    if (a->rank != b->rank || a->size != b->size) return fail(TN_ERROR, "allclose: shapes differ");
    if (a->environment.kind != TN_DEVICE || b->environment.kind != TN_DEVICE ||
        a->environment.resource.device.id != b->environment.resource.device.id)
        return fail(TN_INCOMPATIBLE_DEVICES, "operands must live on one device");
    TN_TRY(use_device_of(a));
    PairGeom g;
    make_geom(a, b, a, g);
    cudaStream_t s = as_cuda(stream);
    *close = 1;
    if (g.n == 0) return TN_SUCCESS;
    int* flag = nullptr;
    TN_TRY(scratch_alloc(reinterpret_cast<void**>(&flag), sizeof(int), s));
    cudaError_t err = cudaMemsetAsync(flag, 0, sizeof(int), s);
    if (err == cudaSuccess) {
        const int grid = grid_for(g.n);
        switch (a->dtype) {
            case TN_FLOAT16: allclose_kernel<__half><<<grid, kThreads, 0, s>>>(static_cast<const __half*>(a->address), static_cast<const __half*>(b->address), g, rtol, atol, flag); break;
            case TN_BFLOAT16: allclose_kernel<__nv_bfloat16><<<grid, kThreads, 0, s>>>(static_cast<const __nv_bfloat16*>(a->address), static_cast<const __nv_bfloat16*>(b->address), g, rtol, atol, flag); break;
            case TN_FLOAT32: allclose_kernel<float><<<grid, kThreads, 0, s>>>(static_cast<const float*>(a->address), static_cast<const float*>(b->address), g, rtol, atol, flag); break;
            default: allclose_kernel<double><<<grid, kThreads, 0, s>>>(static_cast<const double*>(a->address), static_cast<const double*>(b->address), g, rtol, atol, flag); break;
        }
        count_launch();
        err = cudaGetLastError();
    }
    int mismatch = 0;
    if (err == cudaSuccess) err = cudaMemcpyAsync(&mismatch, flag, sizeof(int), cudaMemcpyDeviceToHost, s);
    if (err == cudaSuccess) err = cudaStreamSynchronize(s);
    scratch_free(flag, s);
    if (err != cudaSuccess) return fail(TN_ERROR, "allclose failed: %s", cudaGetErrorString(err));
    *close = mismatch ? 0 : 1;
    return surface_device_aborts();
}

tn_status tn_eq(const tn_tensor_t* a, const tn_tensor_t* b, tn_tensor_t* dst, tn_stream_t stream) { return compare_entry<CMP_EQ>(a, b, dst, stream); }
tn_status tn_ne(const tn_tensor_t* a, const tn_tensor_t* b, tn_tensor_t* dst, tn_stream_t stream) { return compare_entry<CMP_NE>(a, b, dst, stream); }
tn_status tn_gt(const tn_tensor_t* a, const tn_tensor_t* b, tn_tensor_t* dst, tn_stream_t stream) { return compare_entry<CMP_GT>(a, b, dst, stream); }
tn_status tn_ge(const tn_tensor_t* a, const tn_tensor_t* b, tn_tensor_t* dst, tn_stream_t stream) { return compare_entry<CMP_GE>(a, b, dst, stream); }
tn_status tn_lt(const tn_tensor_t* a, const tn_tensor_t* b, tn_tensor_t* dst, tn_stream_t stream) { return compare_entry<CMP_LT>(a, b, dst, stream); }
tn_status tn_le(const tn_tensor_t* a, const tn_tensor_t* b, tn_tensor_t* dst, tn_stream_t stream) { return compare_entry<CMP_LE>(a, b, dst, stream); }

}  // extern "C"
