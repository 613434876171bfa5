// Data-movement operators around the hot path: outer product, repeat, concat, triangular
// masks and the two complex constructors. They replace src/cuda/outer.cu, reps.cu, concat.cu,
// traing.cu and complex.cu of the reference. Outer, repeat and concat are expressed as views
// over the existing broadcast multiply and strided copy; the other two have kernels here.
#include "common.cuh"

namespace tnb {
namespace {

constexpr int kThreads = 256;

int grid_for(int64_t n) {
    const int64_t cap = (int64_t)sm_count() * 8;
    int64_t blocks = ceil_div(n, kThreads);
    if (blocks < 1) blocks = 1;
    return (int)(blocks < cap ? blocks : cap);
}

bool on_one_device(const tn_tensor_t* a, const tn_tensor_t* b) {
    return a->environment.kind == TN_DEVICE && b->environment.kind == TN_DEVICE &&
           a->environment.resource.device.id == b->environment.resource.device.id;
}

// A view record over `base`'s storage with the given shape and element strides.
tn_tensor_t view_of(const tn_tensor_t* base, void* address, int rank, const int64_t* sizes, const int64_t* strides) {
    tn_tensor_t v = *base;
    v.address = address;
    v.rank = (uint8_t)rank;
    size_t n = 1;
    for (int d = 0; d < TN_MAX_RANK; ++d) {
        v.shape.sizes[d] = d < rank ? (size_t)sizes[d] : 0;
        v.strides.sizes[d] = d < rank ? strides[d] : 0;
        if (d < rank) n *= (size_t)sizes[d];
    }
    v.size = n;
    v.layout = TN_STRIDED;
    return v;
}

void dense_strides(int rank, const int64_t* sizes, int64_t* strides) {
    int64_t run = 1;
    for (int d = rank - 1; d >= 0; --d) {
        strides[d] = run;
        run *= sizes[d];
    }
}

// dst[i][j] = keep(i, j) ? src[i][j] : 0, elements moved as raw words (zero is all-zero bits for
// every supported type). Upper keeps j >= i + k, lower keeps j <= i + k, in signed arithmetic.
template <typename W, bool UPPER>
__global__ void __launch_bounds__(kThreads) triangular(const W* __restrict__ src, W* __restrict__ dst, int64_t rows, int64_t cols,
                                                       int64_t ss0, int64_t ss1, int64_t ds0, int64_t ds1, int64_t k) {
    const int64_t n = rows * cols;
    const int64_t step = (int64_t)gridDim.x * kThreads;
    for (int64_t lin = (int64_t)blockIdx.x * kThreads + threadIdx.x; lin < n; lin += step) {
        const int64_t i = lin / cols, j = lin - i * cols;
        const bool keep = UPPER ? (j >= i + k) : (j <= i + k);
        W v = W();
        if (keep) v = src[i * ss0 + j * ss1];
        dst[i * ds0 + j * ds1] = v;
    }
}

struct ComplexGeom {
    int rank;
    int64_t n;
    int64_t sizes[TN_MAX_RANK];
    int64_t sa[TN_MAX_RANK];
    int64_t sb[TN_MAX_RANK];
    int dt_a, dt_b;
};

// dst (interleaved re, im; written densely in logical order) from two real tensors with
// size-1 broadcasting: (a, b) as they are, or (a cos b, a sin b).
template <typename F, bool POLAR>
__global__ void __launch_bounds__(kThreads) complex_from_pair(const void* __restrict__ a, const void* __restrict__ b, F* __restrict__ dst,
                                                              const __grid_constant__ ComplexGeom g) {
    const int64_t step = (int64_t)gridDim.x * kThreads;
    for (int64_t lin = (int64_t)blockIdx.x * kThreads + threadIdx.x; lin < g.n; lin += step) {
        int64_t rest = lin, oa = 0, ob = 0;
        for (int d = g.rank - 1; d >= 0; --d) {
            const int64_t c = rest % g.sizes[d];
            rest /= g.sizes[d];
            oa += c * g.sa[d];
            ob += c * g.sb[d];
        }
        const F x = load_as<F>(a, g.dt_a, oa), y = load_as<F>(b, g.dt_b, ob);
        F re, im;
        if constexpr (POLAR) {
            F s, c;
            if constexpr (std::is_same<F, float>::value) sincosf(y, &s, &c);
            else sincos(y, &s, &c);
            re = x * c;
            im = x * s;
        } else {
            re = x;
            im = y;
        }
        dst[2 * lin] = re;
        dst[2 * lin + 1] = im;
    }
}

template <bool POLAR>
tn_status complex_view(const tn_tensor_t* a, const tn_tensor_t* b, tn_tensor_t* dst, tn_stream_t stream, const char* what) {
    if (!a || !b || !dst) return fail(TN_ERROR, "null tensor");
    if (!on_one_device(a, dst) || !on_one_device(b, dst)) return fail(TN_INCOMPATIBLE_DEVICES, "operands must live on one device");
    auto real_kind = [](int dt) { return is_int(dt) || dt == TN_FLOAT32 || dt == TN_FLOAT64; };
    if (!real_kind(a->dtype) || !real_kind(b->dtype)) return fail(TN_UNSUPPORTED_DTYPE, "%s: operand dtypes %d, %d", what, (int)a->dtype, (int)b->dtype);
    const bool wide = a->dtype == TN_FLOAT64 || b->dtype == TN_FLOAT64;
    if (!POLAR && (is_int(a->dtype) || is_int(b->dtype))) return fail(TN_UNSUPPORTED_DTYPE, "%s: integer parts", what);
    if (dst->dtype != (wide ? TN_COMPLEX128 : TN_COMPLEX64))
        return fail(TN_UNSUPPORTED_DTYPE, "%s: result dtype %d for %s parts", what, (int)dst->dtype, wide ? "float64" : "float32");
    if (a->rank != dst->rank || b->rank != dst->rank) return fail(TN_ERROR, "%s: ranks differ", what);
    TN_TRY(use_device_of(dst));
    ComplexGeom g = {};
    g.rank = dst->rank;
    g.n = 1;
    for (int d = 0; d < g.rank; ++d) {
        g.sizes[d] = (int64_t)dst->shape.sizes[d];
        g.n *= g.sizes[d];
        if ((a->shape.sizes[d] != 1 && a->shape.sizes[d] != dst->shape.sizes[d]) || (b->shape.sizes[d] != 1 && b->shape.sizes[d] != dst->shape.sizes[d]))
            return fail(TN_ERROR, "%s: shapes do not broadcast", what);
        g.sa[d] = a->shape.sizes[d] == 1 ? 0 : a->strides.sizes[d];
        g.sb[d] = b->shape.sizes[d] == 1 ? 0 : b->strides.sizes[d];
    }
    g.dt_a = a->dtype;
    g.dt_b = b->dtype;
    if (g.n == 0) return TN_SUCCESS;
    cudaStream_t s = as_cuda(stream);
    const int grid = grid_for(g.n);
    if (wide) complex_from_pair<double, POLAR><<<grid, kThreads, 0, s>>>(a->address, b->address, static_cast<double*>(dst->address), g);
    else complex_from_pair<float, POLAR><<<grid, kThreads, 0, s>>>(a->address, b->address, static_cast<float*>(dst->address), g);
    return after_launch(what);
}

template <bool UPPER>
tn_status triangular_op(const tn_tensor_t* src, tn_tensor_t* dst, tn_stream_t stream, int k, const char* what) {
    if (!src || !dst) return fail(TN_ERROR, "null tensor");
    if (!on_one_device(src, dst)) return fail(TN_INCOMPATIBLE_DEVICES, "operands must live on one device");
    if (src->rank != 2 || dst->rank != 2) return fail(TN_UNSUPPORTED_DTYPE, "%s: rank %d (matrices only)", what, (int)src->rank);
    if (src->dtype != dst->dtype || !is_numeric(src->dtype)) return fail(TN_UNSUPPORTED_DTYPE, "%s: dtypes %d -> %d", what, (int)src->dtype, (int)dst->dtype);
    if (src->shape.sizes[0] != dst->shape.sizes[0] || src->shape.sizes[1] != dst->shape.sizes[1]) return fail(TN_ERROR, "%s: shapes differ", what);
    TN_TRY(use_device_of(dst));
    const int64_t rows = (int64_t)src->shape.sizes[0], cols = (int64_t)src->shape.sizes[1];
    if (rows * cols == 0) return TN_SUCCESS;
    cudaStream_t s = as_cuda(stream);
    const int grid = grid_for(rows * cols);
    const int64_t ss0 = src->strides.sizes[0], ss1 = src->strides.sizes[1], ds0 = dst->strides.sizes[0], ds1 = dst->strides.sizes[1];
    switch (dtype_bytes(src->dtype)) {
        case 1: triangular<uint8_t, UPPER><<<grid, kThreads, 0, s>>>(static_cast<const uint8_t*>(src->address), static_cast<uint8_t*>(dst->address), rows, cols, ss0, ss1, ds0, ds1, k); break;
        case 2: triangular<uint16_t, UPPER><<<grid, kThreads, 0, s>>>(static_cast<const uint16_t*>(src->address), static_cast<uint16_t*>(dst->address), rows, cols, ss0, ss1, ds0, ds1, k); break;
        case 4: triangular<uint32_t, UPPER><<<grid, kThreads, 0, s>>>(static_cast<const uint32_t*>(src->address), static_cast<uint32_t*>(dst->address), rows, cols, ss0, ss1, ds0, ds1, k); break;
        default: triangular<uint64_t, UPPER><<<grid, kThreads, 0, s>>>(static_cast<const uint64_t*>(src->address), static_cast<uint64_t*>(dst->address), rows, cols, ss0, ss1, ds0, ds1, k); break;
    }
    return after_launch(what);
}

}  // namespace
}  // namespace tnb

using namespace tnb;

extern "C" {

tn_status tn_outer(const tn_tensor_t* a, const tn_tensor_t* b, tn_tensor_t* dst, tn_stream_t stream) {
    if (!a || !b || !dst) return fail(TN_ERROR, "null tensor");
    if (a->rank != 1 || b->rank != 1 || dst->rank != 2) return fail(TN_ERROR, "outer: vectors in, matrix out");
    if (dst->shape.sizes[0] != a->shape.sizes[0] || dst->shape.sizes[1] != b->shape.sizes[0]) return fail(TN_ERROR, "outer: result shape");
    // a[:, None] * b[None, :] through the broadcast multiply
    const int64_t sa[2] = {(int64_t)a->shape.sizes[0], 1}, sta[2] = {a->strides.sizes[0], 0};
    const int64_t sb[2] = {1, (int64_t)b->shape.sizes[0]}, stb[2] = {0, b->strides.sizes[0]};
    const tn_tensor_t va = view_of(a, a->address, 2, sa, sta), vb = view_of(b, b->address, 2, sb, stb);
    return tn_mul(&va, &vb, dst, stream);
}

tn_status tn_repeat(const tn_tensor_t* src, tn_tensor_t* dst, int axis, int reps, tn_stream_t stream) {
    if (!src || !dst) return fail(TN_ERROR, "null tensor");
    const int R = src->rank;
    if (R < 1 || axis < 0 || axis >= R || reps < 1) return fail(TN_ERROR, "repeat: axis %d, reps %d for rank %d", axis, reps, R);
    if (R >= TN_MAX_RANK) return fail(TN_ERROR, "repeat: rank %d leaves no spare dimension", R);
    if (dst->rank != R || dst->dtype != src->dtype) return fail(TN_UNSUPPORTED_DTYPE, "repeat: result rank or dtype");
    // every element of the axis `reps` times in a row: a copy from a view with one more dimension
    // of extent `reps` and stride 0, into the dense result seen with the same extra dimension
    int64_t sizes[TN_MAX_RANK], ssrc[TN_MAX_RANK], sdst[TN_MAX_RANK];
    int n = 0;
    for (int d = 0; d < R; ++d) {
        sizes[n] = (int64_t)src->shape.sizes[d];
        ssrc[n] = src->strides.sizes[d];
        ++n;
        if (d == axis) {
            sizes[n] = reps;
            ssrc[n] = 0;
            ++n;
        }
        if (dst->shape.sizes[d] != src->shape.sizes[d] * (d == axis ? (size_t)reps : 1)) return fail(TN_ERROR, "repeat: result shape");
    }
    dense_strides(n, sizes, sdst);
    const tn_tensor_t vs = view_of(src, src->address, n, sizes, ssrc);
    tn_tensor_t vd = view_of(dst, dst->address, n, sizes, sdst);
    return tn_cpy(&vs, &vd, stream);
}

tn_status tn_concat(const tn_tensor_t* a, const tn_tensor_t* b, tn_tensor_t* dst, tn_stream_t stream, int axis) {
    if (!a || !b || !dst) return fail(TN_ERROR, "null tensor");
    const int R = dst->rank;
    if (a->rank != R || b->rank != R || axis < 0 || axis >= R) return fail(TN_ERROR, "concat: ranks / axis");
    if (a->dtype != dst->dtype || b->dtype != dst->dtype) return fail(TN_UNSUPPORTED_DTYPE, "concat: dtypes %d, %d -> %d", (int)a->dtype, (int)b->dtype, (int)dst->dtype);
    int64_t sizes[TN_MAX_RANK], sdst[TN_MAX_RANK], sa[TN_MAX_RANK], sb[TN_MAX_RANK];
    for (int d = 0; d < R; ++d) {
        sizes[d] = (int64_t)dst->shape.sizes[d];
        sa[d] = (int64_t)a->shape.sizes[d];
        sb[d] = (int64_t)b->shape.sizes[d];
        if (d == axis ? sa[d] + sb[d] != sizes[d] : (sa[d] != sizes[d] || sb[d] != sizes[d])) return fail(TN_ERROR, "concat: shapes");
    }
    // the result is written densely: each operand is a strided copy into its slab of it
    dense_strides(R, sizes, sdst);
    tn_tensor_t da = view_of(dst, dst->address, R, sa, sdst);
    void* second = static_cast<unsigned char*>(dst->address) + (size_t)(sa[axis] * sdst[axis]) * dtype_bytes(dst->dtype);
    tn_tensor_t db = view_of(dst, second, R, sb, sdst);
    if (da.size) TN_TRY(tn_cpy(a, &da, stream));
    if (db.size) TN_TRY(tn_cpy(b, &db, stream));
    return TN_SUCCESS;
}

tn_status tn_triu(const tn_tensor_t* src, tn_tensor_t* dst, tn_stream_t stream, int k) { return triangular_op<true>(src, dst, stream, k, "triu"); }
tn_status tn_tril(const tn_tensor_t* src, tn_tensor_t* dst, tn_stream_t stream, int k) { return triangular_op<false>(src, dst, stream, k, "tril"); }

tn_status tn_view_as_cartesian(const tn_tensor_t* re, const tn_tensor_t* im, tn_tensor_t* dst, tn_stream_t stream) {
    return complex_view<false>(re, im, dst, stream, "view_as_cartesian");
}
tn_status tn_view_as_polar(const tn_tensor_t* rho, const tn_tensor_t* theta, tn_tensor_t* dst, tn_stream_t stream) {
    return complex_view<true>(rho, theta, dst, stream, "view_as_polar");
}

}  // extern "C"
