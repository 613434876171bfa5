// Elementwise family: add/sub/mul/pow with NumPy broadcast, the unary math functions, scale,
// and the fused elementwise program. Replaces src/cuda/ops-binary.cu, ops-unary.cu, ops-scale.cu
// of the reference.
//
// Three kernels stream HBM exactly once with 128-bit accesses:
//   ew_flat     both operands dense (or a single broadcast scalar) -> one flat range;
//   ew_rows     dst viewed as [rows, cols]; each operand is dense along cols or constant
//               along cols, with an arbitrary row pitch (covers row- and column-broadcast);
//   ew_program  the same [rows, cols] geometry for up to 4 inputs and a list of nodes.
// Everything else (mixed dtypes, ragged widths, arbitrary strided views) goes through
// ew_generic, which decodes the linear index per element.
#include "common.cuh"
#include "eltwise_program.cuh"
#include "eltwise_jit.cuh"

#include <mutex>
#include <vector>

#include <cmath>
#include <cstdlib>
#include <cstring>

namespace tnb {
namespace {

using namespace prog;
static_assert(sizeof(tn_eltwise_node_t) == 8 && offsetof(tn_eltwise_node_t, imm) == 4, "the run-time compiler's copy of the node layout");

template <typename T, int OP>
__device__ __forceinline__ Vec<T> apply_vec(const Vec<T>& a, const Vec<T>& b, Imm imm) {
    using C = typename compute_of<T>::type;
    constexpr bool FAST = sizeof(T) == 2;
    Vec<T> d;
#pragma unroll
    for (int i = 0; i < Vec<T>::N; ++i)
        d.e[i] = from_compute<T, C>(apply_op<OP, FAST, C>(to_compute<C>(a.e[i]), to_compute<C>(b.e[i]), imm));
    return d;
}

template <typename T, int OP>
__device__ __forceinline__ T apply_one(T a, T b, Imm imm) {
    using C = typename compute_of<T>::type;
    constexpr bool FAST = sizeof(T) == 2;
    return from_compute<T, C>(apply_op<OP, FAST, C>(to_compute<C>(a), to_compute<C>(b), imm));
}

// ------------------------------------------------------------------ ew_flat -----------
// d[i] = op(a[i*sa], b[i*sb]) for i < n with sa, sb in {0, 1}. Vector body + scalar tail.
template <typename T, int OP>
__global__ void __launch_bounds__(kThreads) ew_flat(const T* __restrict__ a, const T* __restrict__ b,
                                                    T* __restrict__ d, int64_t n, int sa, int sb, Imm imm) {
    constexpr int V = Vec<T>::N;
    constexpr int UNROLL = 4;
    constexpr bool BIN = op_is_binary(OP);
    const int64_t nvec = n / V;
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    const int64_t tid = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    Vec<T> ca, cb;
    if (sa == 0) ca = splat_vec(a[0]);
    if (BIN && sb == 0) cb = splat_vec(b[0]);
    int64_t i = tid;
    for (; i + (UNROLL - 1) * stride < nvec; i += UNROLL * stride) {
        Vec<T> va[UNROLL], vb[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int64_t off = (i + u * stride) * V;
            va[u] = sa ? load_vec(a + off) : ca;
            if (BIN) vb[u] = sb ? load_vec(b + off) : cb;
            else vb[u] = va[u];
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) store_vec(d + (i + u * stride) * V, apply_vec<T, OP>(va[u], vb[u], imm));
    }
    for (; i < nvec; i += stride) {
        Vec<T> va = sa ? load_vec(a + i * V) : ca;
        Vec<T> vb = BIN ? (sb ? load_vec(b + i * V) : cb) : va;
        store_vec(d + i * V, apply_vec<T, OP>(va, vb, imm));
    }
    const int64_t tail = nvec * V + tid;
    if (tail < n) {
        T x = a[sa ? tail : 0];
        T y = BIN ? b[sb ? tail : 0] : x;
        d[tail] = apply_one<T, OP>(x, y, imm);
    }
}

// ------------------------------------------------------------------ ew_rows -----------
// dst is [rows, cols] dense. A vector operand X contributes the 16 bytes at X + r * x_rs + c
// (x_rs == 0 for a row-broadcast operand: the same vector every row, served by L1); a SCALAR
// operand contributes X[r * x_rs] to the whole row (column-broadcast). A thread owns one column
// slot and walks down the rows, UNROLL adjacent rows at a time, with every load of the group
// issued before the first use. The load path has no data-dependent branch: operand kinds are
// template parameters, so the compiler keeps all loads of a group in flight together.
struct RowsGeom {
    int64_t rows, cols;
    int64_t a_rs, b_rs;
};

template <typename T, int OP, bool A_SCALAR, bool B_SCALAR>
__global__ void __launch_bounds__(kThreads) ew_rows(const T* __restrict__ a, const T* __restrict__ b,
                                                    T* __restrict__ d, RowsGeom g, Imm imm) {
    constexpr int V = Vec<T>::N;
    constexpr int UNROLL = 4;
    constexpr bool BIN = op_is_binary(OP);
    const int64_t cvec = g.cols / V;
    const int64_t rstep = (int64_t)gridDim.y * UNROLL;
    for (int64_t cv = (int64_t)blockIdx.x * kThreads + threadIdx.x; cv < cvec; cv += (int64_t)gridDim.x * kThreads) {
        const int64_t c = cv * V;
        for (int64_t r0 = (int64_t)blockIdx.y * UNROLL; r0 < g.rows; r0 += rstep) {
            Vec<T> va[UNROLL], vb[UNROLL];
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const int64_t r = r0 + u < g.rows ? r0 + u : g.rows - 1;  // the tail re-reads the last row
                if constexpr (A_SCALAR) va[u] = splat_vec(__ldg(a + r * g.a_rs));
                else va[u] = load_vec(a + r * g.a_rs + c);
                if constexpr (!BIN) vb[u] = va[u];
                else if constexpr (B_SCALAR) vb[u] = splat_vec(__ldg(b + r * g.b_rs));
                else vb[u] = load_vec(b + r * g.b_rs + c);
            }
#pragma unroll
            for (int u = 0; u < UNROLL; ++u)
                if (r0 + u < g.rows) store_vec(d + (r0 + u) * g.cols + c, apply_vec<T, OP>(va[u], vb[u], imm));
        }
    }
}

// ------------------------------------------------------------------ ew_generic --------
struct GenericArgs {
    const void* a;
    const void* b;
    void* d;
    int adt, bdt, ddt;
    int rank;
    int64_t n;
    int64_t sizes[TN_MAX_RANK];
    int64_t sa[TN_MAX_RANK];
    int64_t sb[TN_MAX_RANK];
    Imm imm;
};

template <typename C, int OP, typename I>
__global__ void __launch_bounds__(kThreads) ew_generic(GenericArgs g) {
    const I n = static_cast<I>(g.n);
    const I step = static_cast<I>(gridDim.x) * kThreads;
    for (I lin = static_cast<I>(blockIdx.x) * kThreads + threadIdx.x; lin < n; lin += step) {
        I rem = lin;
        int64_t oa = 0, ob = 0;
        for (int dim = g.rank - 1; dim >= 0; --dim) {
            const I size = static_cast<I>(g.sizes[dim]);
            const I coord = rem % size;
            rem /= size;
            oa += static_cast<int64_t>(coord) * g.sa[dim];
            ob += static_cast<int64_t>(coord) * g.sb[dim];
        }
        C x = load_as<C>(g.a, g.adt, oa);
        C y = op_is_binary(OP) ? load_as<C>(g.b, g.bdt, ob) : x;
        store_as<C>(g.d, g.ddt, static_cast<int64_t>(lin), apply_op<OP, false, C>(x, y, g.imm));
    }
}

// ------------------------------------------------------------------ host planning ------
// Broadcast-aligned, size-1-free, coalesced view of the operands over dst's logical shape.
struct Plan {
    int rank = 0;
    int64_t n = 1;
    int64_t sizes[TN_MAX_RANK] = {0};
    int64_t st[TN_PROGRAM_MAX_INPUTS][TN_MAX_RANK] = {{0}};
};

tn_status build_plan(const tn_tensor_t* const* ops, int nops, const tn_tensor_t* dst, Plan& plan) {
    const int R = dst->rank;
    if (R > TN_MAX_RANK) return fail(TN_ERROR, "rank %d exceeds %d", R, TN_MAX_RANK);
    int64_t sizes[TN_MAX_RANK];
    int64_t st[TN_PROGRAM_MAX_INPUTS][TN_MAX_RANK];
    int64_t n = 1;
    for (int d = 0; d < R; ++d) {
        sizes[d] = (int64_t)dst->shape.sizes[d];
        n *= sizes[d];
    }
    for (int k = 0; k < nops; ++k) {
        const tn_tensor_t* t = ops[k];
        if (t->rank > R) return fail(TN_ERROR, "operand rank %d exceeds result rank %d", (int)t->rank, R);
        const int off = R - t->rank;
        for (int d = 0; d < R; ++d) {
            if (d < off) { st[k][d] = 0; continue; }
            const int64_t sz = (int64_t)t->shape.sizes[d - off];
            if (sz != 1 && sz != sizes[d])
                return fail(TN_ERROR, "operand extent %lld does not broadcast to %lld at dim %d",
                            (long long)sz, (long long)sizes[d], d);
            st[k][d] = sz == 1 ? 0 : t->strides.sizes[d - off];
        }
    }
    // drop extent-1 dims, then merge neighbours that every operand walks contiguously
    int r = 0;
    for (int d = 0; d < R; ++d) {
        if (sizes[d] == 1) continue;
        bool merged = false;
        if (r > 0) {
            merged = true;
            for (int k = 0; k < nops; ++k)
                if (plan.st[k][r - 1] != st[k][d] * sizes[d]) { merged = false; break; }
            if (merged) {
                plan.sizes[r - 1] *= sizes[d];
                for (int k = 0; k < nops; ++k) plan.st[k][r - 1] = st[k][d];
            }
        }
        if (!merged) {
            plan.sizes[r] = sizes[d];
            for (int k = 0; k < nops; ++k) plan.st[k][r] = st[k][d];
            ++r;
        }
    }
    plan.rank = r;
    plan.n = n;
    return TN_SUCCESS;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

inline int env_int(const char* name, int fallback) { return env_knob(name, fallback); }

int flat_grid(int64_t work_items) {
    const int64_t cap = (int64_t)sm_count() * 8;  // 8 CTAs of 256 threads fill an SM
    int64_t blocks = ceil_div(work_items, kThreads);
    if (blocks < 1) blocks = 1;
    return (int)(blocks < cap ? blocks : cap);
}

// CTAs of `kernel` that fit on one SM at once (from the occupancy calculator, cached by the
// caller): grids are sized to exactly one resident wave so that no partial wave trails.
template <typename K>
int resident_ctas(K kernel, int threads, size_t dynamic_smem = 0) {
    // Remembered per (kernel, shared-memory size): kernels of one signature share this function's
    // instantiation, so the cache is keyed by the function pointer, not by the template.
    struct Entry { const void* kernel; size_t smem; int ctas; };
    static std::mutex mutex;
    static std::vector<Entry> seen;
    const void* key = reinterpret_cast<const void*>(kernel);
    std::lock_guard<std::mutex> lock(mutex);
    for (const Entry& e : seen)
        if (e.kernel == key && e.smem == dynamic_smem) return e.ctas;
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, threads, dynamic_smem) != cudaSuccess || n < 1) {
        cudaGetLastError();
        n = 1;
    }
    seen.push_back({key, dynamic_smem, n});
    return n;
}

template <typename T, int OP, bool AS, bool BS>
tn_status launch_rows(const T* pa, const T* pb, T* pd, const RowsGeom& g, Imm imm, cudaStream_t s) {
    constexpr int V = Vec<T>::N;
    static const int per_sm = resident_ctas(ew_rows<T, OP, AS, BS>, kThreads);
    const int64_t cvec = g.cols / V;
    const int64_t cap = (int64_t)sm_count() * per_sm;
    int64_t gx = ceil_div(cvec, kThreads);
    if (gx > cap) gx = cap;
    int64_t gy = cap / gx;
    const int64_t groups = ceil_div(g.rows, 4);
    if (gy > groups) gy = groups;
    if (gy < 1) gy = 1;
    if (gy > 65535) gy = 65535;
    ew_rows<T, OP, AS, BS><<<dim3((unsigned)gx, (unsigned)gy), kThreads, 0, s>>>(pa, pb, pd, g, imm);
    return after_launch("ew_rows");
}

// Launches the fastest kernel that the geometry allows for a same-dtype op.
template <typename T, int OP>
tn_status launch_typed(const Plan& plan, const void* a, const void* b, void* d, Imm imm, cudaStream_t s, bool* done) {
    constexpr int V = Vec<T>::N;
    constexpr bool BIN = op_is_binary(OP);
    *done = false;
    if (plan.n == 0) { *done = true; return TN_SUCCESS; }
    const T* pa = static_cast<const T*>(a);
    const T* pb = static_cast<const T*>(BIN ? b : a);
    T* pd = static_cast<T*>(d);
    if (!aligned16(d)) return TN_SUCCESS;
    if (plan.rank <= 1) {
        const int64_t sa = plan.rank ? plan.st[0][0] : 0;
        const int64_t sb = BIN ? (plan.rank ? plan.st[1][0] : 0) : sa;
        if ((sa != 0 && sa != 1) || (sb != 0 && sb != 1)) return TN_SUCCESS;
        if ((sa == 1 && !aligned16(a)) || (BIN && sb == 1 && !aligned16(b))) return TN_SUCCESS;
        static const int per_sm = resident_ctas(ew_flat<T, OP>, kThreads);
        const int64_t cap = (int64_t)sm_count() * per_sm;
        int64_t grid = ceil_div(ceil_div(plan.n, V), kThreads);
        if (grid > cap) grid = cap;
        if (grid < 1) grid = 1;
        ew_flat<T, OP><<<(unsigned)grid, kThreads, 0, s>>>(pa, pb, pd, plan.n, (int)sa, (int)sb, imm);
        *done = true;
        return after_launch("ew_flat");
    }
    if (plan.rank == 2) {
        RowsGeom g;
        g.rows = plan.sizes[0];
        g.cols = plan.sizes[1];
        g.a_rs = plan.st[0][0];
        g.b_rs = BIN ? plan.st[1][0] : g.a_rs;
        const int64_t a_in = plan.st[0][1], b_in = BIN ? plan.st[1][1] : a_in;
        if (g.cols % V) return TN_SUCCESS;
        if ((a_in != 0 && a_in != 1) || (b_in != 0 && b_in != 1)) return TN_SUCCESS;
        if (g.a_rs < 0 || g.b_rs < 0) return TN_SUCCESS;
        if (a_in && (!aligned16(a) || g.a_rs % V)) return TN_SUCCESS;
        if (BIN && b_in && (!aligned16(b) || g.b_rs % V)) return TN_SUCCESS;
        if (!a_in && !b_in) return TN_SUCCESS;  // both column-broadcast: generic path
        *done = true;
        if constexpr (BIN) {
            if (!a_in) return launch_rows<T, OP, true, false>(pa, pb, pd, g, imm, s);
            if (!b_in) return launch_rows<T, OP, false, true>(pa, pb, pd, g, imm, s);
        } else {
            if (!a_in) { *done = false; return TN_SUCCESS; }
        }
        return launch_rows<T, OP, false, false>(pa, pb, pd, g, imm, s);
    }
    return TN_SUCCESS;
}

template <typename C, int OP>
tn_status launch_generic(const Plan& plan, const tn_tensor_t* a, const tn_tensor_t* b, tn_tensor_t* dst, Imm imm,
                         cudaStream_t s) {
    if (plan.n == 0) return TN_SUCCESS;
    GenericArgs g;
    g.a = a->address;
    g.b = b ? b->address : a->address;
    g.d = dst->address;
    g.adt = a->dtype;
    g.bdt = b ? b->dtype : a->dtype;
    g.ddt = dst->dtype;
    g.rank = plan.rank;
    g.n = plan.n;
    for (int d = 0; d < plan.rank; ++d) {
        g.sizes[d] = plan.sizes[d];
        g.sa[d] = plan.st[0][d];
        g.sb[d] = b ? plan.st[1][d] : plan.st[0][d];
    }
    g.imm = imm;
    const int grid = flat_grid(plan.n);
    if (plan.n < (int64_t(1) << 31)) ew_generic<C, OP, uint32_t><<<grid, kThreads, 0, s>>>(g);
    else ew_generic<C, OP, uint64_t><<<grid, kThreads, 0, s>>>(g);
    return after_launch("ew_generic");
}

// ---- complex64 / complex128 (same-type add, sub, mul; neg and repack) -------------------------
// The reference's tables hold complex entries for exactly these (src/cpu/ops-binary.cpp:222-223 and
// the Sub / Mul twins; src/cpu/ops-unary.cpp:214-215,232-233). An element is a (re, im) pair of
// F; the kernel decodes the logical index like ew_generic.
template <typename F, int OP, typename I>
__global__ void __launch_bounds__(kThreads) ew_complex(GenericArgs g) {
    const I n = static_cast<I>(g.n);
    const I step = static_cast<I>(gridDim.x) * kThreads;
    for (I lin = static_cast<I>(blockIdx.x) * kThreads + threadIdx.x; lin < n; lin += step) {
        I rem = lin;
        int64_t oa = 0, ob = 0;
        for (int dim = g.rank - 1; dim >= 0; --dim) {
            const I size = static_cast<I>(g.sizes[dim]);
            const I coord = rem % size;
            rem /= size;
            oa += static_cast<int64_t>(coord) * g.sa[dim];
            ob += static_cast<int64_t>(coord) * g.sb[dim];
        }
        const F xr = static_cast<const F*>(g.a)[2 * oa], xi = static_cast<const F*>(g.a)[2 * oa + 1];
        const F yr = static_cast<const F*>(g.b)[2 * ob], yi = static_cast<const F*>(g.b)[2 * ob + 1];
        F rr, ri;
        if constexpr (OP == TN_OP_ADD) { rr = xr + yr; ri = xi + yi; }
        else if constexpr (OP == TN_OP_SUB) { rr = xr - yr; ri = xi - yi; }
        else if constexpr (OP == TN_OP_MUL) { rr = xr * yr - xi * yi; ri = xr * yi + xi * yr; }
        else if constexpr (OP == TN_OP_NEG) { rr = -xr; ri = -xi; }
        else { rr = xr; ri = xi; }
        static_cast<F*>(g.d)[2 * static_cast<int64_t>(lin)] = rr;
        static_cast<F*>(g.d)[2 * static_cast<int64_t>(lin) + 1] = ri;
    }
}

inline bool is_complex(int dt) { return dt == TN_COMPLEX64 || dt == TN_COMPLEX128; }

template <int OP>
tn_status launch_complex(const Plan& plan, const tn_tensor_t* a, const tn_tensor_t* b, tn_tensor_t* dst, cudaStream_t s) {
    if constexpr (OP == TN_OP_ADD || OP == TN_OP_SUB || OP == TN_OP_MUL || OP == TN_OP_NEG || OP == TN_OP_COUNT) {
        if (plan.n == 0) return TN_SUCCESS;
        GenericArgs g;
        g.a = a->address;
        g.b = b ? b->address : a->address;
        g.d = dst->address;
        g.adt = g.bdt = g.ddt = a->dtype;
        g.rank = plan.rank;
        g.n = plan.n;
        for (int d = 0; d < plan.rank; ++d) {
            g.sizes[d] = plan.sizes[d];
            g.sa[d] = plan.st[0][d];
            g.sb[d] = b ? plan.st[1][d] : plan.st[0][d];
        }
        g.imm = Imm{0.0, 0};
        const int grid = flat_grid(plan.n);
        const bool small = plan.n < (int64_t(1) << 31);
        if (a->dtype == TN_COMPLEX64) {
            if (small) ew_complex<float, OP, uint32_t><<<grid, kThreads, 0, s>>>(g);
            else ew_complex<float, OP, uint64_t><<<grid, kThreads, 0, s>>>(g);
        } else {
            if (small) ew_complex<double, OP, uint32_t><<<grid, kThreads, 0, s>>>(g);
            else ew_complex<double, OP, uint64_t><<<grid, kThreads, 0, s>>>(g);
        }
        return after_launch("ew_complex");
    } else {
        return fail(TN_UNSUPPORTED_DTYPE, "operation %d has no complex form", OP);
    }
}

// Arithmetic class of a dtype pair (mirrors the result types of the reference's tables,
// src/cpu/ops-binary.cpp:168-430): 0 = int64 wrap, 1 = float32, 2 = float64.
int compute_class(int a, int b) {
    if (a == TN_FLOAT64 || b == TN_FLOAT64) return 2;
    const bool fa = is_float(a), fb = is_float(b);
    if ((fa && b == TN_INT64) || (fb && a == TN_INT64)) return 2;
    if (fa || fb) return 1;
    return 0;
}

// Pairs the reference accepts (src/cpu/ops-binary.cpp:168-430); everything else is
// TN_UNSUPPORTED_DTYPE, exactly as its default table entry.
bool pair_supported(int op, int a, int b) {
    if (!is_numeric(a) || !is_numeric(b)) return false;
    if (is_int(a) && is_int(b)) return op != TN_OP_POW;
    auto half_ok = [](int h, int o) { return o == h || o == TN_FLOAT32 || o == TN_FLOAT64 || is_int(o); };
    if (is_half(a)) return half_ok(a, b);
    if (is_half(b)) return half_ok(b, a);
    auto wide_ok = [](int o) { return o == TN_FLOAT32 || o == TN_FLOAT64 || o == TN_INT32; };
    return wide_ok(a) && wide_ok(b);
}

template <int OP>
tn_status typed_dispatch(int dt, const Plan& plan, const void* a, const void* b, void* d, Imm imm, cudaStream_t s,
                         bool* done) {
    switch (dt) {
        case TN_FLOAT16: return launch_typed<__half, OP>(plan, a, b, d, imm, s, done);
        case TN_BFLOAT16: return launch_typed<__nv_bfloat16, OP>(plan, a, b, d, imm, s, done);
        case TN_FLOAT32: return launch_typed<float, OP>(plan, a, b, d, imm, s, done);
        case TN_FLOAT64: return launch_typed<double, OP>(plan, a, b, d, imm, s, done);
        default: break;
    }
    if constexpr (!op_is_float_only(OP)) {
        switch (dt) {
            case TN_INT8: return launch_typed<int8_t, OP>(plan, a, b, d, imm, s, done);
            case TN_INT16: return launch_typed<int16_t, OP>(plan, a, b, d, imm, s, done);
            case TN_INT32: return launch_typed<int32_t, OP>(plan, a, b, d, imm, s, done);
            case TN_INT64: return launch_typed<int64_t, OP>(plan, a, b, d, imm, s, done);
            default: break;
        }
    }
    *done = false;
    return TN_SUCCESS;
}

template <int OP>
tn_status generic_dispatch(int cls, const Plan& plan, const tn_tensor_t* a, const tn_tensor_t* b, tn_tensor_t* dst,
                           Imm imm, cudaStream_t s) {
    if (cls == 2) return launch_generic<double, OP>(plan, a, b, dst, imm, s);
    if (cls == 1) return launch_generic<float, OP>(plan, a, b, dst, imm, s);
    if constexpr (!op_is_float_only(OP)) return launch_generic<int64_t, OP>(plan, a, b, dst, imm, s);
    return fail(TN_UNSUPPORTED_DTYPE, "operation needs a floating dtype");
}

// Dense operands of two different types (float16 + float32, float32 + float64, int32 + float32, ...):
// eight elements per thread and iteration through 16-byte loads, computed in the wider type like the
// element-wise kernel, which takes every other mixed case.
template <typename T>
__device__ __forceinline__ void load8(const T* p, T (&v)[8]) {
    constexpr int CHUNKS = 8 * sizeof(T) / 16;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) reinterpret_cast<uint4*>(v)[c] = __ldg(reinterpret_cast<const uint4*>(p) + c);
}
template <typename T>
__device__ __forceinline__ void store8(T* p, const T (&v)[8]) {
    constexpr int CHUNKS = 8 * sizeof(T) / 16;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) reinterpret_cast<uint4*>(p)[c] = reinterpret_cast<const uint4*>(v)[c];
}

template <typename TA, typename TB, typename TD, typename C, int OP>
__global__ void __launch_bounds__(kThreads) ew_flat_mixed(const TA* __restrict__ a, const TB* __restrict__ b, TD* __restrict__ d, int64_t n, Imm imm) {
    const int64_t groups = n / 8;
    const int64_t step = (int64_t)gridDim.x * kThreads;
    for (int64_t g = (int64_t)blockIdx.x * kThreads + threadIdx.x; g < groups; g += step) {
        alignas(16) TA va[8];
        alignas(16) TB vb[8];
        alignas(16) TD vd[8];
        load8(a + g * 8, va);
        load8(b + g * 8, vb);
#pragma unroll
        for (int k = 0; k < 8; ++k) vd[k] = from_compute<TD, C>(apply_op<OP, false, C>(to_compute<C>(va[k]), to_compute<C>(vb[k]), imm));
        store8(d + g * 8, vd);
    }
    if (blockIdx.x == 0 && threadIdx.x < n - groups * 8) {
        const int64_t i = groups * 8 + threadIdx.x;
        d[i] = from_compute<TD, C>(apply_op<OP, false, C>(to_compute<C>(a[i]), to_compute<C>(b[i]), imm));
    }
}

template <typename TA, typename TB, typename TD, typename C, int OP>
tn_status launch_flat_mixed(const void* a, const void* b, void* d, int64_t n, Imm imm, cudaStream_t s) {
    ew_flat_mixed<TA, TB, TD, C, OP><<<flat_grid(ceil_div(n, 8)), kThreads, 0, s>>>(static_cast<const TA*>(a), static_cast<const TB*>(b),
                                                                                static_cast<TD*>(d), n, imm);
    return after_launch("ew_flat_mixed");
}

// Returns TN_UNSUPPORTED_DTYPE when the triple is not one of the compiled ones (the caller goes on).
template <int OP>
tn_status flat_mixed_dispatch(int adt, int bdt, int ddt, const void* a, const void* b, void* d, int64_t n, Imm imm, cudaStream_t s) {
#define TN_MIXED(A_DT, B_DT, D_DT, TA, TB, TD, C) \
    if (adt == A_DT && bdt == B_DT && ddt == D_DT) return launch_flat_mixed<TA, TB, TD, C, OP>(a, b, d, n, imm, s);
    TN_MIXED(TN_FLOAT16, TN_FLOAT32, TN_FLOAT32, __half, float, float, float)
    TN_MIXED(TN_FLOAT32, TN_FLOAT16, TN_FLOAT32, float, __half, float, float)
    TN_MIXED(TN_BFLOAT16, TN_FLOAT32, TN_FLOAT32, __nv_bfloat16, float, float, float)
    TN_MIXED(TN_FLOAT32, TN_BFLOAT16, TN_FLOAT32, float, __nv_bfloat16, float, float)
    TN_MIXED(TN_FLOAT32, TN_FLOAT64, TN_FLOAT64, float, double, double, double)
    TN_MIXED(TN_FLOAT64, TN_FLOAT32, TN_FLOAT64, double, float, double, double)
    TN_MIXED(TN_INT32, TN_FLOAT32, TN_FLOAT32, int32_t, float, float, float)
    TN_MIXED(TN_FLOAT32, TN_INT32, TN_FLOAT32, float, int32_t, float, float)
#undef TN_MIXED
    return TN_UNSUPPORTED_DTYPE;
}

// Large same-type operations whose operands are strided views of the full result shape (transposes,
// permutes, strided slices) would take the element-by-element kernel at about 1 TB/s. Copying such an
// operand dense first (tiled transposes, 16-byte runs: about 3 TB/s) and then taking the vector
// kernel is faster in total, so that is what happens above 2^20 elements.
bool is_dense(const tn_tensor_t* t) {
    int64_t expect = 1;
    for (int d = t->rank - 1; d >= 0; --d) {
        if (t->shape.sizes[d] != 1 && t->strides.sizes[d] != expect) return false;
        expect *= (int64_t)t->shape.sizes[d];
    }
    return true;
}
bool full_strided_view(const tn_tensor_t* t, const tn_tensor_t* dst) {
    if (t->rank != dst->rank || t->size != dst->size || is_dense(t)) return false;
    // worth copying only if the copy itself is fast: some dimension of the view is contiguous (runs that
    // move as 16-byte words, or a tiled transpose); a view with no unit stride (every second column,
    // say) copies element by element and is better read in place (measured: 1.06 against 0.53 TB/s)
    bool unit = false;
    for (int d = 0; d < t->rank; ++d) {
        if (t->shape.sizes[d] != dst->shape.sizes[d]) return false;
        if (t->strides.sizes[d] == 1 && t->shape.sizes[d] >= 16) unit = true;
    }
    return unit;
}
tn_status densify(const tn_tensor_t* t, tn_tensor_t* out, void** mem, tn_stream_t stream) {
    *out = *t;
    int64_t run = 1;
    for (int d = t->rank - 1; d >= 0; --d) {
        out->strides.sizes[d] = run;
        run *= (int64_t)t->shape.sizes[d];
    }
    out->layout = TN_CONTIGUOUS;
    TN_TRY(scratch_alloc(mem, (size_t)run * dtype_bytes(t->dtype), as_cuda(stream)));
    out->address = *mem;
    return tn_cpy(t, out, stream);
}
constexpr size_t kDensifyFrom = size_t(1) << 20;

template <int OP>
tn_status binary(const tn_tensor_t* a, const tn_tensor_t* b, tn_tensor_t* dst, tn_stream_t stream) {
    if (!a || !b || !dst) return fail(TN_ERROR, "null tensor");
    const bool cplx = is_complex(a->dtype) && a->dtype == b->dtype && dst->dtype == a->dtype && OP != TN_OP_POW;
    if (!cplx && (!pair_supported(OP, a->dtype, b->dtype) || !is_numeric(dst->dtype)))
        return fail(TN_UNSUPPORTED_DTYPE, "binary op %d: dtype pair (%d, %d) -> %d unsupported", OP, (int)a->dtype,
                    (int)b->dtype, (int)dst->dtype);
    if (a->environment.kind != TN_DEVICE || b->environment.kind != TN_DEVICE ||
        a->environment.resource.device.id != b->environment.resource.device.id ||
        a->environment.resource.device.id != dst->environment.resource.device.id)
        return fail(TN_INCOMPATIBLE_DEVICES, "operands must live on one device");
    TN_TRY(use_device_of(dst));
    Plan plan;
    const tn_tensor_t* ops[2] = {a, b};
    TN_TRY(build_plan(ops, 2, dst, plan));
    cudaStream_t s = as_cuda(stream);
    if (cplx) return launch_complex<OP>(plan, a, b, dst, s);
    Imm imm{0.0, 0};
    if (a->dtype == b->dtype && a->dtype == dst->dtype) {
        bool done = false;
        TN_TRY((typed_dispatch<OP>(a->dtype, plan, a->address, b->address, dst->address, imm, s, &done)));
        if (done) return TN_SUCCESS;
        const bool fix_a = full_strided_view(a, dst), fix_b = full_strided_view(b, dst);
        if (dst->size >= kDensifyFrom && is_dense(dst) && (fix_a || fix_b)) {
            tn_tensor_t da, db;
            void *ma = nullptr, *mb = nullptr;
            tn_status st = TN_SUCCESS;
            if (fix_a) st = densify(a, &da, &ma, stream);
            if (st == TN_SUCCESS && fix_b) st = densify(b, &db, &mb, stream);
            if (st == TN_SUCCESS) st = binary<OP>(fix_a ? &da : a, fix_b ? &db : b, dst, stream);
            if (ma) scratch_free(ma, s);
            if (mb) scratch_free(mb, s);
            return st;
        }
    }
    if (a->dtype != b->dtype && plan.n >= 4096 && is_dense(a) && is_dense(b) && is_dense(dst) && a->size == dst->size && b->size == dst->size &&
        ((reinterpret_cast<uintptr_t>(a->address) | reinterpret_cast<uintptr_t>(b->address) | reinterpret_cast<uintptr_t>(dst->address)) & 15) == 0) {
        const tn_status st = flat_mixed_dispatch<OP>(a->dtype, b->dtype, dst->dtype, a->address, b->address, dst->address, plan.n, imm, s);
        if (st != TN_UNSUPPORTED_DTYPE) return st;
    }
    return generic_dispatch<OP>(compute_class(a->dtype, b->dtype), plan, a, b, dst, imm, s);
}

bool unary_supported(int op, int dt) {
    if (op == TN_OP_NEG || op == TN_OP_SCALE || op == TN_OP_COUNT /* repack */) return is_numeric(dt);
    if (op == TN_OP_ABS) return is_float(dt) || dt == TN_INT32 || dt == TN_INT64;  // src/cpu/ops-unary.cpp:288-300
    return is_float(dt);
}

template <int OP>
tn_status unary(const tn_tensor_t* src, tn_tensor_t* dst, tn_stream_t stream, Imm imm) {
    if (!src || !dst) return fail(TN_ERROR, "null tensor");
    const bool cplx = is_complex(src->dtype) && dst->dtype == src->dtype && (OP == TN_OP_NEG || OP == TN_OP_COUNT);
    if (!cplx && (!unary_supported(OP, src->dtype) || !is_numeric(dst->dtype)))
        return fail(TN_UNSUPPORTED_DTYPE, "unary op %d: dtype %d unsupported", OP, (int)src->dtype);
    if (src->environment.kind != TN_DEVICE ||
        src->environment.resource.device.id != dst->environment.resource.device.id)
        return fail(TN_INCOMPATIBLE_DEVICES, "operands must live on one device");
    TN_TRY(use_device_of(dst));
    Plan plan;
    const tn_tensor_t* ops[1] = {src};
    TN_TRY(build_plan(ops, 1, dst, plan));
    cudaStream_t s = as_cuda(stream);
    if (cplx) return launch_complex<OP>(plan, src, nullptr, dst, s);
    if (src->dtype == dst->dtype) {
        bool done = false;
        TN_TRY((typed_dispatch<OP>(src->dtype, plan, src->address, nullptr, dst->address, imm, s, &done)));
        if (done) return TN_SUCCESS;
        if (OP != TN_OP_COUNT && dst->size >= kDensifyFrom && is_dense(dst) && full_strided_view(src, dst)) {
            tn_tensor_t dense;
            void* mem = nullptr;
            tn_status st = densify(src, &dense, &mem, stream);
            if (st == TN_SUCCESS) st = unary<OP>(&dense, dst, stream, imm);
            if (mem) scratch_free(mem, s);
            return st;
        }
    }
    const int cls = src->dtype == TN_FLOAT64 ? 2 : (is_float(src->dtype) ? 1 : 0);
    return generic_dispatch<OP>(cls, plan, src, nullptr, dst, imm, s);
}

// Reads a host scalar of dtype `dt` (reference: scalar_t, include/tannic/runtime/tensor.h:43-46).
bool read_scalar(const tn_scalar_t* sc, Imm* imm) {
    const void* p = sc->address;
    switch (sc->dtype) {
        case TN_INT8: imm->i = *static_cast<const int8_t*>(p); break;
        case TN_INT16: imm->i = *static_cast<const int16_t*>(p); break;
        case TN_INT32: imm->i = *static_cast<const int32_t*>(p); break;
        case TN_INT64: imm->i = *static_cast<const int64_t*>(p); break;
        case TN_FLOAT16: { __half h; memcpy(&h, p, 2); imm->f = __half2float(h); break; }
        case TN_BFLOAT16: { __nv_bfloat16 h; memcpy(&h, p, 2); imm->f = __bfloat162float(h); break; }
        case TN_FLOAT32: imm->f = *static_cast<const float*>(p); break;
        case TN_FLOAT64: imm->f = *static_cast<const double*>(p); break;
        default: return false;
    }
    if (is_int(sc->dtype)) imm->f = (double)imm->i;
    else imm->i = (int64_t)imm->f;
    return true;
}

// ------------------------------------------------------------------ fused program ------
struct ProgGenericArgs {
    const void* in[kMaxIn];
    void* d;
    int rank;
    int64_t n;
    int64_t sizes[TN_MAX_RANK];
    int64_t st[kMaxIn][TN_MAX_RANK];
    int n_inputs, n_nodes;
    tn_eltwise_node_t nodes[kMaxNodes];
};

template <typename T>
__global__ void __launch_bounds__(kThreads) ew_program_generic(const __grid_constant__ ProgGenericArgs g) {
    using C = typename compute_of<T>::type;
    constexpr bool FAST = sizeof(T) == 2;
    const int64_t step = (int64_t)gridDim.x * kThreads;
    for (int64_t lin = (int64_t)blockIdx.x * kThreads + threadIdx.x; lin < g.n; lin += step) {
        int64_t rem = lin;
        int64_t off[kMaxIn] = {0, 0, 0, 0};
        for (int dim = g.rank - 1; dim >= 0; --dim) {
            const int64_t coord = rem % g.sizes[dim];
            rem /= g.sizes[dim];
#pragma unroll
            for (int k = 0; k < kMaxIn; ++k) off[k] += coord * g.st[k][dim];
        }
        C val[kMaxIn + kMaxNodes];
#pragma unroll
        for (int k = 0; k < kMaxIn; ++k)
            val[k] = k < g.n_inputs ? to_compute<C>(static_cast<const T*>(g.in[k])[off[k]]) : C(0);
        for (int n = 0; n < g.n_nodes; ++n) {
            const tn_eltwise_node_t nd = g.nodes[n];
            val[kMaxIn + n] = round_to_storage<T, C>(apply_dynamic<C, FAST>(nd.opcode, val[nd.lhs], val[nd.rhs], nd.imm));
        }
        static_cast<T*>(g.d)[lin] = from_compute<T, C>(val[kMaxIn + g.n_nodes - 1]);
    }
}

template <typename P>
bool matches(const tn_eltwise_node_t* nodes, int n) {
    if (n != P::N) return false;
    for (int k = 0; k < n; ++k) {
        const bool bin = op_is_binary(nodes[k].opcode);
        if (nodes[k].opcode != P::nodes[k].op || nodes[k].lhs != P::nodes[k].lhs) return false;
        if (bin && nodes[k].rhs != P::nodes[k].rhs) return false;
    }
    return true;
}

// A program that computes the same expression as a compiled one, with its nodes listed in another
// order, its inputs numbered differently or the operands of an add / multiply swapped, is rewritten
// into the compiled program's own form, so that what reaches the fast path does not depend on how the
// caller walked its expression tree. The two DAGs are unified from the result downwards: node against
// node of the same opcode (both operand orders for the commutative ones, which give bit-identical
// results), input against input. Every node of the caller's program must take part.
template <typename P>
struct Unifier {
    const tn_eltwise_node_t* nodes;
    int n_inputs;
    int node_of[P::N];   // pattern node -> program node
    int input_of[kMaxIn];  // pattern input -> program input

    bool value(int pv, int gv) {
        if (pv < kMaxIn) {
            if (gv >= kMaxIn || gv >= n_inputs) return false;
            if (input_of[pv] >= 0) return input_of[pv] == gv;
            input_of[pv] = gv;
            return true;
        }
        if (gv < kMaxIn) return false;
        return node(pv - kMaxIn, gv - kMaxIn);
    }
    bool node(int pk, int gk) {
        if (node_of[pk] >= 0) return node_of[pk] == gk;
        const NodeSpec want = P::nodes[pk];
        const tn_eltwise_node_t& got = nodes[gk];
        if (got.opcode != want.op) return false;
        const Unifier saved = *this;
        node_of[pk] = gk;
        if (!op_is_binary(want.op)) {
            if (value(want.lhs, got.lhs)) return true;
            *this = saved;
            return false;
        }
        if (value(want.lhs, got.lhs) && value(want.rhs, got.rhs)) return true;
        *this = saved;
        if (want.op == TN_OP_ADD || want.op == TN_OP_MUL) {
            node_of[pk] = gk;
            if (value(want.lhs, got.rhs) && value(want.rhs, got.lhs)) return true;
            *this = saved;
        }
        return false;
    }
};

// On success `nodes` holds the compiled program's node list (immediates carried over) and `inputs`
// its inputs in the compiled program's numbering.
template <typename P>
bool rewrite_as(tn_eltwise_node_t* nodes, int n_nodes, const tn_tensor_t** inputs, int* n_inputs) {
    if (n_nodes != P::N) return false;
    Unifier<P> u;
    u.nodes = nodes;
    u.n_inputs = *n_inputs;
    for (int k = 0; k < P::N; ++k) u.node_of[k] = -1;
    for (int k = 0; k < kMaxIn; ++k) u.input_of[k] = -1;
    if (!u.node(P::N - 1, n_nodes - 1)) return false;
    bool used[kMaxNodes] = {};
    for (int k = 0; k < P::N; ++k) {
        if (u.node_of[k] < 0 || used[u.node_of[k]]) return false;
        used[u.node_of[k]] = true;
    }
    for (int k = 0; k < P::NIN; ++k)
        if (u.input_of[k] < 0) return false;
    tn_eltwise_node_t out[P::N];
    const tn_tensor_t* in[kMaxIn] = {};
    for (int k = 0; k < P::N; ++k) {
        out[k] = nodes[u.node_of[k]];
        out[k].lhs = static_cast<uint8_t>(P::nodes[k].lhs);
        out[k].rhs = static_cast<uint8_t>(op_is_binary(P::nodes[k].op) ? P::nodes[k].rhs : P::nodes[k].lhs);
    }
    for (int k = 0; k < P::NIN; ++k) in[k] = inputs[u.input_of[k]];
    for (int k = 0; k < P::N; ++k) nodes[k] = out[k];
    for (int k = 0; k < P::NIN; ++k) inputs[k] = in[k];
    *n_inputs = P::NIN;
    return true;
}

bool rewrite_as_compiled(tn_eltwise_node_t* nodes, int n_nodes, const tn_tensor_t** inputs, int* n_inputs) {
    return rewrite_as<ProgLogSquareExp>(nodes, n_nodes, inputs, n_inputs) || rewrite_as<ProgMulAdd>(nodes, n_nodes, inputs, n_inputs) ||
           rewrite_as<ProgSquaredDiff>(nodes, n_nodes, inputs, n_inputs) || rewrite_as<ProgNormScale>(nodes, n_nodes, inputs, n_inputs);
}

template <typename T>
tn_status launch_program(const Plan& plan, const tn_tensor_t* const* inputs, int n_inputs,
                         const tn_eltwise_node_t* nodes, int n_nodes, tn_tensor_t* dst, cudaStream_t s) {
    constexpr int V = Vec<T>::N;
    if (plan.n == 0) return TN_SUCCESS;
    // [rows, cols] geometry?
    bool rows_ok = plan.rank <= 2 && aligned16(dst->address);
    const int64_t rows = plan.rank == 2 ? plan.sizes[0] : 1;
    const int64_t cols = plan.rank == 0 ? 1 : plan.sizes[plan.rank - 1];
    if (cols % V) rows_ok = false;
    for (int k = 0; rows_ok && k < n_inputs; ++k) {
        const int64_t inner = plan.rank ? plan.st[k][plan.rank - 1] : 0;
        const int64_t rs = plan.rank == 2 ? plan.st[k][0] : 0;
        if ((inner != 0 && inner != 1) || rs < 0) rows_ok = false;
        if (inner == 1 && (!aligned16(inputs[k]->address) || rs % V)) rows_ok = false;
    }
    if (rows_ok) {
        ProgArgs g;
        memset(&g, 0, sizeof(g));
        for (int k = 0; k < n_inputs; ++k) {
            g.in[k] = inputs[k]->address;
            g.inner[k] = plan.rank ? (int)plan.st[k][plan.rank - 1] : 0;
            g.rs[k] = plan.rank == 2 ? plan.st[k][0] : 0;
        }
        g.d = dst->address;
        g.rows = rows;
        g.cols = cols;
        g.n_inputs = n_inputs;
        g.n_nodes = n_nodes;
        for (int k = 0; k < n_nodes; ++k) g.nodes[k] = nodes[k];
        bool any_scalar = false;
        for (int k = 0; k < n_inputs; ++k) any_scalar = any_scalar || g.inner[k] == 0;
        const int unroll = env_int("TN_PROGRAM_UNROLL", 2);
        // one resident wave: CTAs per SM from the occupancy calculator (remembered per kernel and shared-memory size)
        auto launch = [&](auto kernel, int u, size_t smem = 0) {
            const int per_sm = resident_ctas(kernel, kThreads, smem);
            const int64_t cvec = cols / V;
            // two resident waves' worth of CTAs measured a few percent faster than exactly one
            const int64_t cap = (int64_t)sm_count() * env_int("TN_PROGRAM_CTAS_PER_SM", 2 * per_sm);
            int64_t gx = ceil_div(cvec, kThreads);
            if (gx > cap) gx = cap;
            int64_t gy = cap / gx;
            const int64_t groups = ceil_div(rows, u);
            if (gy > groups) gy = groups;
            if (gy < 1) gy = 1;
            if (gy > 65535) gy = 65535;
            kernel<<<dim3((unsigned)gx, (unsigned)gy), kThreads, smem, s>>>(g);
        };
#define TN_LAUNCH_PROGRAM(PROG)                                                         \
    do {                                                                                \
        if (any_scalar) launch(ew_program_rows<T, PROG, 1, true>, 1);                   \
        else if (unroll >= 4) launch(ew_program_rows<T, PROG, 4, false>, 4);            \
        else if (unroll >= 2) launch(ew_program_rows<T, PROG, 2, false>, 2);            \
        else launch(ew_program_rows<T, PROG, 1, false>, 1);                             \
    } while (0)
        if (matches<ProgLogSquareExp>(nodes, n_nodes)) TN_LAUNCH_PROGRAM(ProgLogSquareExp);
        else if (matches<ProgMulAdd>(nodes, n_nodes)) TN_LAUNCH_PROGRAM(ProgMulAdd);
        else if (matches<ProgSquaredDiff>(nodes, n_nodes)) TN_LAUNCH_PROGRAM(ProgSquaredDiff);
        else if (matches<ProgNormScale>(nodes, n_nodes)) TN_LAUNCH_PROGRAM(ProgNormScale);
        else if (const JitKernel* jit = jit_program_rows(dtype_of<T>::value, nodes, n_nodes, n_inputs, any_scalar ? 1 : (unroll >= 4 ? 4 : unroll >= 2 ? 2 : 1),
                                                        any_scalar, plan.n)) {
            // the caller's own program, instantiated at run time: same kernel template, same launch geometry
            const int u = any_scalar ? 1 : (unroll >= 4 ? 4 : unroll >= 2 ? 2 : 1);
            const int64_t cvec = cols / V;
            const int64_t cap = (int64_t)sm_count() * env_int("TN_PROGRAM_CTAS_PER_SM", 2 * jit->ctas_per_sm);
            int64_t gx = ceil_div(cvec, kThreads);
            if (gx > cap) gx = cap;
            int64_t gy = cap / gx;
            const int64_t groups = ceil_div(rows, u);
            if (gy > groups) gy = groups;
            if (gy < 1) gy = 1;
            if (gy > 65535) gy = 65535;
            return jit_launch(jit, (unsigned)gx, (unsigned)gy, &g, s);
        } else {
            // the interpreter: 16 bytes of shared memory per thread and value
            // two vectors per dispatch measured no faster than one (2.64 against 2.74 TB/s): one is the default
            const int iu = any_scalar ? 1 : (env_int("TN_INTERPRETER_UNROLL", 1) >= 2 ? 2 : 1);
            const size_t smem = (size_t)(kMaxIn + n_nodes) * kThreads * 16 * iu;
            static thread_local int attr_device = -1;
            int dev = 0;
            TN_CUDA(cudaGetDevice(&dev));
            if (attr_device != dev) {
                const int most = (kMaxIn + kMaxNodes) * kThreads * 16 * 2;
                TN_CUDA(cudaFuncSetAttribute(ew_program_rows<T, ProgDynamic, 1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, most));
                TN_CUDA(cudaFuncSetAttribute(ew_program_rows<T, ProgDynamic, 1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, most));
                TN_CUDA(cudaFuncSetAttribute(ew_program_rows<T, ProgDynamic, 2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, most));
                attr_device = dev;
            }
            if (any_scalar) launch(ew_program_rows<T, ProgDynamic, 1, true>, 1, smem);
            else if (iu == 2) launch(ew_program_rows<T, ProgDynamic, 2, false>, 2, smem);
            else launch(ew_program_rows<T, ProgDynamic, 1, false>, 1, smem);
        }
#undef TN_LAUNCH_PROGRAM
        return after_launch("ew_program_rows");
    }
    ProgGenericArgs g;
    memset(&g, 0, sizeof(g));
    for (int k = 0; k < n_inputs; ++k) {
        g.in[k] = inputs[k]->address;
        for (int d = 0; d < plan.rank; ++d) g.st[k][d] = plan.st[k][d];
    }
    g.d = dst->address;
    g.rank = plan.rank;
    g.n = plan.n;
    for (int d = 0; d < plan.rank; ++d) g.sizes[d] = plan.sizes[d];
    g.n_inputs = n_inputs;
    g.n_nodes = n_nodes;
    for (int k = 0; k < n_nodes; ++k) g.nodes[k] = nodes[k];
    ew_program_generic<T><<<flat_grid(plan.n), kThreads, 0, s>>>(g);
    return after_launch("ew_program_generic");
}

}  // namespace

bool read_host_scalar(const tn_scalar_t* sc, double* f, int64_t* i) {
    Imm imm{0.0, 0};
    if (!sc || !sc->address || !read_scalar(sc, &imm)) return false;
    *f = imm.f;
    *i = imm.i;
    return true;
}

}  // namespace tnb

using namespace tnb;

extern "C" {

tn_status tn_add(const tn_tensor_t* a, const tn_tensor_t* b, tn_tensor_t* d, tn_stream_t s) { return binary<TN_OP_ADD>(a, b, d, s); }
tn_status tn_sub(const tn_tensor_t* a, const tn_tensor_t* b, tn_tensor_t* d, tn_stream_t s) { return binary<TN_OP_SUB>(a, b, d, s); }
tn_status tn_mul(const tn_tensor_t* a, const tn_tensor_t* b, tn_tensor_t* d, tn_stream_t s) { return binary<TN_OP_MUL>(a, b, d, s); }
tn_status tn_pow(const tn_tensor_t* a, const tn_tensor_t* b, tn_tensor_t* d, tn_stream_t s) { return binary<TN_OP_POW>(a, b, d, s); }

tn_status tn_neg(const tn_tensor_t* x, tn_tensor_t* d, tn_stream_t s) { return unary<TN_OP_NEG>(x, d, s, Imm{0, 0}); }
tn_status tn_repack(const tn_tensor_t* x, tn_tensor_t* d, tn_stream_t s) {
    // a strided view goes through the copy machinery (coalesced dimensions, 16-byte runs, tiled
    // transposes); a dense source keeps the flat path
    if (x && d && x->dtype == d->dtype && x->rank == d->rank && x->rank > 0) {
        bool dense = true, same = true;
        int64_t expect = 1;
        for (int dim = x->rank - 1; dim >= 0; --dim) {
            if (x->shape.sizes[dim] != d->shape.sizes[dim]) same = false;
            if (x->shape.sizes[dim] != 1 && x->strides.sizes[dim] != expect) dense = false;
            expect *= (int64_t)x->shape.sizes[dim];
        }
        if (same && !dense) return tn_cpy(x, d, s);
    }
    return unary<TN_OP_COUNT>(x, d, s, Imm{0, 0});
}
tn_status tn_log(const tn_tensor_t* x, tn_tensor_t* d, tn_stream_t s) { return unary<TN_OP_LOG>(x, d, s, Imm{0, 0}); }
tn_status tn_exp(const tn_tensor_t* x, tn_tensor_t* d, tn_stream_t s) { return unary<TN_OP_EXP>(x, d, s, Imm{0, 0}); }
tn_status tn_sqrt(const tn_tensor_t* x, tn_tensor_t* d, tn_stream_t s) { return unary<TN_OP_SQRT>(x, d, s, Imm{0, 0}); }
tn_status tn_rsqrt(const tn_tensor_t* x, tn_tensor_t* d, tn_stream_t s, float eps) { return unary<TN_OP_RSQRT>(x, d, s, Imm{(double)eps, 0}); }
tn_status tn_abs(const tn_tensor_t* x, tn_tensor_t* d, tn_stream_t s) { return unary<TN_OP_ABS>(x, d, s, Imm{0, 0}); }
tn_status tn_sin(const tn_tensor_t* x, tn_tensor_t* d, tn_stream_t s) { return unary<TN_OP_SIN>(x, d, s, Imm{0, 0}); }
tn_status tn_cos(const tn_tensor_t* x, tn_tensor_t* d, tn_stream_t s) { return unary<TN_OP_COS>(x, d, s, Imm{0, 0}); }
tn_status tn_tan(const tn_tensor_t* x, tn_tensor_t* d, tn_stream_t s) { return unary<TN_OP_TAN>(x, d, s, Imm{0, 0}); }
tn_status tn_sinh(const tn_tensor_t* x, tn_tensor_t* d, tn_stream_t s) { return unary<TN_OP_SINH>(x, d, s, Imm{0, 0}); }
tn_status tn_cosh(const tn_tensor_t* x, tn_tensor_t* d, tn_stream_t s) { return unary<TN_OP_COSH>(x, d, s, Imm{0, 0}); }
tn_status tn_tanh(const tn_tensor_t* x, tn_tensor_t* d, tn_stream_t s) { return unary<TN_OP_TANH>(x, d, s, Imm{0, 0}); }

tn_status tn_scale(const tn_tensor_t* src, const tn_scalar_t* scalar, tn_tensor_t* dst, tn_stream_t stream) {
    if (!src || !scalar || !dst) return fail(TN_ERROR, "null argument");
    // same-dtype only, as the reference's table (src/cpu/ops-scale.cpp:103-114)
    if (scalar->dtype != src->dtype || !is_numeric(src->dtype))
        return fail(TN_UNSUPPORTED_DTYPE, "scale: tensor dtype %d, scalar dtype %d", (int)src->dtype, (int)scalar->dtype);
    Imm imm{0.0, 0};
    if (!scalar->address || !read_scalar(scalar, &imm)) return fail(TN_ERROR, "scale: unreadable scalar");
    return unary<TN_OP_SCALE>(src, dst, stream, imm);
}

tn_status tn_eltwise_program(const tn_tensor_t* const* inputs, int n_inputs, const tn_eltwise_node_t* nodes,
                             int n_nodes, tn_tensor_t* dst, tn_stream_t stream) {
    if (!inputs || !nodes || !dst) return fail(TN_ERROR, "null argument");
    if (n_inputs < 1 || n_inputs > TN_PROGRAM_MAX_INPUTS || n_nodes < 1 || n_nodes > TN_PROGRAM_MAX_NODES)
        return fail(TN_ERROR, "program with %d inputs / %d nodes is out of range", n_inputs, n_nodes);
    const int dt = dst->dtype;
    if (!is_float(dt)) return fail(TN_UNSUPPORTED_DTYPE, "fused programs run on floating dtypes, got %d", dt);
    for (int k = 0; k < n_inputs; ++k) {
        if (!inputs[k]) return fail(TN_ERROR, "null input %d", k);
        if (inputs[k]->dtype != dt) return fail(TN_UNSUPPORTED_DTYPE, "input %d has dtype %d, result has %d", k, (int)inputs[k]->dtype, dt);
        if (inputs[k]->environment.kind != TN_DEVICE ||
            inputs[k]->environment.resource.device.id != dst->environment.resource.device.id)
            return fail(TN_INCOMPATIBLE_DEVICES, "operands must live on one device");
    }
    for (int k = 0; k < n_nodes; ++k) {
        const tn_eltwise_node_t& nd = nodes[k];
        if (nd.opcode >= TN_OP_COUNT) return fail(TN_ERROR, "node %d: unknown opcode %d", k, (int)nd.opcode);
        auto ok = [&](int v) { return v < n_inputs || (v >= TN_PROGRAM_MAX_INPUTS && v < TN_PROGRAM_MAX_INPUTS + k); };
        if (!ok(nd.lhs) || (op_is_binary(nd.opcode) && !ok(nd.rhs)))
            return fail(TN_ERROR, "node %d reads a value that is not defined before it", k);
    }
    TN_TRY(use_device_of(dst));
    // unary nodes read only lhs; normalise rhs so the kernels may index it blindly
    tn_eltwise_node_t local[TN_PROGRAM_MAX_NODES];
    for (int k = 0; k < n_nodes; ++k) {
        local[k] = nodes[k];
        if (!op_is_binary(local[k].opcode)) local[k].rhs = local[k].lhs;
        // `tensor * scalar` casts the scalar to the tensor's dtype first
        // (include/tannic/operations.hpp:295-313): do the same to a SCALE node's factor
        if (local[k].opcode == TN_OP_SCALE) {
            if (dt == TN_FLOAT16) local[k].imm = __half2float(__float2half_rn(local[k].imm));
            else if (dt == TN_BFLOAT16) local[k].imm = __bfloat162float(__float2bfloat16_rn(local[k].imm));
        }
    }
    // an expression that a compiled program computes takes that program's form, whatever order the
    // caller listed its nodes and inputs in
    const tn_tensor_t* ordered[TN_PROGRAM_MAX_INPUTS] = {};
    for (int k = 0; k < n_inputs; ++k) ordered[k] = inputs[k];
    static const bool no_rewrite = getenv("TN_PROGRAM_NO_REWRITE") != nullptr;
    if (!no_rewrite) rewrite_as_compiled(local, n_nodes, ordered, &n_inputs);
    inputs = ordered;
    Plan plan;
    TN_TRY(build_plan(inputs, n_inputs, dst, plan));
    cudaStream_t s = as_cuda(stream);
    switch (dt) {
        case TN_FLOAT16: return launch_program<__half>(plan, inputs, n_inputs, local, n_nodes, dst, s);
        case TN_BFLOAT16: return launch_program<__nv_bfloat16>(plan, inputs, n_inputs, local, n_nodes, dst, s);
        case TN_FLOAT32: return launch_program<float>(plan, inputs, n_inputs, local, n_nodes, dst, s);
        default: return launch_program<double>(plan, inputs, n_inputs, local, n_nodes, dst, s);
    }
}

}  // extern "C"
