// Device side of the fused element-wise programs: the per-operation arithmetic, 16-byte vectors,
// the compile-time ("static") and interpreted evaluators and the row kernel that runs them.
// eltwise.cu includes this file; the same text is handed to the run-time compiler, which
// instantiates ew_program_rows for a caller's node list (eltwise_jit.cu). It therefore uses
// tnb::stdx (std or cuda::std) and no host header; under the run-time compiler the opcode values
// and program limits arrive as -D definitions generated from the public header's enum.
#pragma once

#include "numeric.cuh"

#ifdef __CUDACC_RTC__
// layout of tn_eltwise_node_t in the public C header (checked against it in eltwise.cu)
struct tn_eltwise_node_t {
    uint8_t opcode;
    uint8_t lhs;
    uint8_t rhs;
    float imm;
};
#else
#include "tannic_b200.h"
#endif

namespace tnb {
namespace prog {

constexpr int kThreads = 256;

struct Imm {
    double f;
    int64_t i;
};

// ------------------------------------------------------------------ the operations ----
template <int OP, bool FAST, typename C>
__device__ __forceinline__ C apply_op(C a, C b, Imm imm) {
    if constexpr (stdx::is_floating_point<C>::value) {
        // Every node rounds on its own: the _rn intrinsics are never contracted into an FMA
        // with a neighbouring node of a fused program.
        if constexpr (stdx::is_same<C, float>::value) {
            if constexpr (OP == TN_OP_ADD) return __fadd_rn(a, b);
            else if constexpr (OP == TN_OP_SUB) return __fsub_rn(a, b);
            else if constexpr (OP == TN_OP_MUL) return __fmul_rn(a, b);
            else if constexpr (OP == TN_OP_SCALE) return __fmul_rn(a, static_cast<float>(imm.f));
        } else {
            if constexpr (OP == TN_OP_ADD) return __dadd_rn(a, b);
            else if constexpr (OP == TN_OP_SUB) return __dsub_rn(a, b);
            else if constexpr (OP == TN_OP_MUL) return __dmul_rn(a, b);
            else if constexpr (OP == TN_OP_SCALE) return __dmul_rn(a, imm.f);
        }
        if constexpr (OP == TN_OP_ADD || OP == TN_OP_SUB || OP == TN_OP_MUL || OP == TN_OP_SCALE) return a;
        else if constexpr (OP == TN_OP_NEG) return -a;
        else if constexpr (OP == TN_OP_ABS) return fabs(a);
        else if constexpr (stdx::is_same<C, float>::value) {
            if constexpr (OP == TN_OP_POW) return powf(a, b);
            else if constexpr (OP == TN_OP_LOG) return FAST ? __logf(a) : logf(a);
            else if constexpr (OP == TN_OP_EXP) return FAST ? __expf(a) : expf(a);
            else if constexpr (OP == TN_OP_SQRT) return sqrtf(a);
            else if constexpr (OP == TN_OP_RSQRT) {
                // The reference evaluates 1.0 / sqrt(x + eps) in double and narrows once
                // (src/cpu/ops-unary.cpp:138-146); half storage is insensitive to it.
                if constexpr (FAST) return rsqrtf(a + static_cast<float>(imm.f));  // one special-function op; 2 ulp in float32, invisible after rounding to 16 bits
                else return static_cast<float>(1.0 / sqrt(static_cast<double>(a) + imm.f));
            }
            else if constexpr (OP == TN_OP_SIN) return sinf(a);
            else if constexpr (OP == TN_OP_COS) return cosf(a);
            else if constexpr (OP == TN_OP_TAN) return tanf(a);
            else if constexpr (OP == TN_OP_SINH) return sinhf(a);
            else if constexpr (OP == TN_OP_COSH) return coshf(a);
            else if constexpr (OP == TN_OP_TANH) {
                if constexpr (FAST) {
                    // 16-bit storage: the special-function unit's tanh (relative error 2^-11) instead of the
                    // twenty-instruction float32 routine; the result is rounded to 8 or 11 significant bits anyway
                    float r;
                    asm("tanh.approx.f32 %0, %1;" : "=f"(r) : "f"(a));
                    return r;
                } else {
                    return tanhf(a);
                }
            }
            else return a;
        } else {
            if constexpr (OP == TN_OP_POW) return pow(a, b);
            else if constexpr (OP == TN_OP_LOG) return log(a);
            else if constexpr (OP == TN_OP_EXP) return exp(a);
            else if constexpr (OP == TN_OP_SQRT) return sqrt(a);
            else if constexpr (OP == TN_OP_RSQRT) return 1.0 / sqrt(a + imm.f);
            else if constexpr (OP == TN_OP_SIN) return sin(a);
            else if constexpr (OP == TN_OP_COS) return cos(a);
            else if constexpr (OP == TN_OP_TAN) return tan(a);
            else if constexpr (OP == TN_OP_SINH) return sinh(a);
            else if constexpr (OP == TN_OP_COSH) return cosh(a);
            else if constexpr (OP == TN_OP_TANH) return tanh(a);
            else return a;
        }
    } else {
        // Integers wrap modulo 2^n: do the arithmetic unsigned, narrow on store.
        using U = typename stdx::make_unsigned<C>::type;
        U x = static_cast<U>(a), y = static_cast<U>(b);
        if constexpr (OP == TN_OP_ADD) return static_cast<C>(x + y);
        else if constexpr (OP == TN_OP_SUB) return static_cast<C>(x - y);
        else if constexpr (OP == TN_OP_MUL) return static_cast<C>(x * y);
        else if constexpr (OP == TN_OP_SCALE) return static_cast<C>(x * static_cast<U>(imm.i));
        else if constexpr (OP == TN_OP_NEG) return static_cast<C>(U(0) - x);
        else if constexpr (OP == TN_OP_ABS) return a < 0 ? static_cast<C>(U(0) - x) : a;
        else return a;
    }
}

__host__ __device__ constexpr bool op_is_binary(int op) { return op <= TN_OP_POW; }
__host__ __device__ constexpr bool op_is_float_only(int op) {
    return op == TN_OP_POW || (op >= TN_OP_LOG && op <= TN_OP_TANH && op != TN_OP_ABS);
}

template <typename T> struct alignas(16) Vec {
    static constexpr int N = 16 / sizeof(T);
    T e[N];
};

template <typename T>
__device__ __forceinline__ Vec<T> load_vec(const T* p) {
    Vec<T> v;
    *reinterpret_cast<uint4*>(&v) = __ldg(reinterpret_cast<const uint4*>(p));
    return v;
}
template <typename T>
__device__ __forceinline__ void store_vec(T* p, const Vec<T>& v) {
    *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(&v);
}
template <typename T>
__device__ __forceinline__ Vec<T> splat_vec(T s) {
    Vec<T> v;
#pragma unroll
    for (int i = 0; i < Vec<T>::N; ++i) v.e[i] = s;
    return v;
}

// ------------------------------------------------------------------ fused program ------
// One pass over HBM for a whole expression tree. Values 0..3 are the inputs, value 4+k is the
// result of node k; every node result is rounded to the storage type T before it is reused,
// which is what the reference's one-kernel-per-node chain does through its temporaries.
constexpr int kMaxIn = TN_PROGRAM_MAX_INPUTS;
constexpr int kMaxNodes = TN_PROGRAM_MAX_NODES;

struct ProgArgs {
    const void* in[kMaxIn];
    void* d;
    int64_t rs[kMaxIn];  // row pitch (elements)
    int inner[kMaxIn];   // 1: dense along cols, 0: constant along cols
    int64_t rows, cols;
    int n_inputs, n_nodes;
    tn_eltwise_node_t nodes[kMaxNodes];
};

template <typename T, typename C>
__device__ __forceinline__ C round_to_storage(C v) {
    if constexpr (stdx::is_same<T, C>::value) return v;
    else return to_compute<C>(from_compute<T, C>(v));
}

template <typename C, bool FAST>
__device__ __forceinline__ C apply_dynamic(int op, C a, C b, float immf) {
    const Imm imm{(double)immf, 0};
    switch (op) {
        case TN_OP_ADD: return apply_op<TN_OP_ADD, FAST, C>(a, b, imm);
        case TN_OP_SUB: return apply_op<TN_OP_SUB, FAST, C>(a, b, imm);
        case TN_OP_MUL: return apply_op<TN_OP_MUL, FAST, C>(a, b, imm);
        case TN_OP_POW: return apply_op<TN_OP_POW, FAST, C>(a, b, imm);
        case TN_OP_NEG: return apply_op<TN_OP_NEG, FAST, C>(a, b, imm);
        case TN_OP_LOG: return apply_op<TN_OP_LOG, FAST, C>(a, b, imm);
        case TN_OP_EXP: return apply_op<TN_OP_EXP, FAST, C>(a, b, imm);
        case TN_OP_SQRT: return apply_op<TN_OP_SQRT, FAST, C>(a, b, imm);
        case TN_OP_RSQRT: return apply_op<TN_OP_RSQRT, FAST, C>(a, b, imm);
        case TN_OP_ABS: return apply_op<TN_OP_ABS, FAST, C>(a, b, imm);
        case TN_OP_SIN: return apply_op<TN_OP_SIN, FAST, C>(a, b, imm);
        case TN_OP_COS: return apply_op<TN_OP_COS, FAST, C>(a, b, imm);
        case TN_OP_TAN: return apply_op<TN_OP_TAN, FAST, C>(a, b, imm);
        case TN_OP_SINH: return apply_op<TN_OP_SINH, FAST, C>(a, b, imm);
        case TN_OP_COSH: return apply_op<TN_OP_COSH, FAST, C>(a, b, imm);
        case TN_OP_TANH: return apply_op<TN_OP_TANH, FAST, C>(a, b, imm);
        case TN_OP_SCALE: return apply_op<TN_OP_SCALE, FAST, C>(a, b, imm);
        default: return a;
    }
}

// Programs compiled ahead of time: the node list is a compile-time constant, so the evaluator
// unrolls into straight-line code with every value in a register. The dynamic evaluator runs
// any other program with its values in local memory.
struct NodeSpec { int op, lhs, rhs; };

struct ProgDynamic { static constexpr int N = 0; static constexpr int NIN = kMaxIn; };

// log(x0) + x1*x1 - exp(x0)
struct ProgLogSquareExp {
    static constexpr int N = 5;
    static constexpr int NIN = 2;
    static constexpr NodeSpec nodes[N] = {{TN_OP_LOG, 0, 0}, {TN_OP_MUL, 1, 1}, {TN_OP_ADD, 4, 5}, {TN_OP_EXP, 0, 0}, {TN_OP_SUB, 6, 7}};
};
// x0*x1 + x2
struct ProgMulAdd {
    static constexpr int N = 2;
    static constexpr int NIN = 3;
    static constexpr NodeSpec nodes[N] = {{TN_OP_MUL, 0, 1}, {TN_OP_ADD, 4, 2}};
};
// (x0 - x1) * (x0 - x1)
struct ProgSquaredDiff {
    static constexpr int N = 2;
    static constexpr int NIN = 2;
    static constexpr NodeSpec nodes[N] = {{TN_OP_SUB, 0, 1}, {TN_OP_MUL, 4, 4}};
};
// x0 * rsqrt(x1, eps) * x2   (normalisation scale)
struct ProgNormScale {
    static constexpr int N = 3;
    static constexpr int NIN = 3;
    static constexpr NodeSpec nodes[N] = {{TN_OP_RSQRT, 1, 1}, {TN_OP_MUL, 0, 4}, {TN_OP_MUL, 5, 2}};
};

template <typename T, typename P, int K, int V, int VALUES>
__device__ __forceinline__ void eval_static(typename compute_of<T>::type (&val)[VALUES][V], const tn_eltwise_node_t* nodes) {
    static_assert(VALUES >= kMaxIn + P::N, "one value per input and node");
    using C = typename compute_of<T>::type;
    constexpr bool FAST = sizeof(T) == 2;
    if constexpr (K < P::N) {
        constexpr NodeSpec nd = P::nodes[K];
        const Imm imm{(double)nodes[K].imm, 0};
#pragma unroll
        for (int i = 0; i < V; ++i)
            val[kMaxIn + K][i] = round_to_storage<T, C>(apply_op<nd.op, FAST, C>(val[nd.lhs][i], val[nd.rhs][i], imm));
        eval_static<T, P, K + 1, V>(val, nodes);
    }
}

// Packed arithmetic for the 16-bit storage types. A native half2 / bfloat162 add, subtract or
// multiply rounds once to the storage type, which is bit-identical to "compute in float32, round
// on store" for these three operations (float32 carries more than twice the significand), so
// such nodes need no conversion at all and process two elements per instruction. The _rn forms
// are never contracted into a fused multiply-add with a neighbouring node.
template <typename T> struct Pack2;
template <> struct Pack2<__half> {
    using type = __half2;
    static __device__ __forceinline__ type add(type a, type b) { return __hadd2_rn(a, b); }
    static __device__ __forceinline__ type sub(type a, type b) { return __hsub2_rn(a, b); }
    static __device__ __forceinline__ type mul(type a, type b) { return __hmul2_rn(a, b); }
    static __device__ __forceinline__ type neg(type a) { return __hneg2(a); }
    static __device__ __forceinline__ type abs(type a) { return __habs2(a); }
    static __device__ __forceinline__ float2 unpack(type a) { return __half22float2(a); }
    static __device__ __forceinline__ type pack(float2 f) { return __float22half2_rn(f); }
    static __device__ __forceinline__ type splat(float f) { return __float2half2_rn(f); }
};
template <> struct Pack2<__nv_bfloat16> {
    using type = __nv_bfloat162;
    static __device__ __forceinline__ type add(type a, type b) { return __hadd2_rn(a, b); }
    static __device__ __forceinline__ type sub(type a, type b) { return __hsub2_rn(a, b); }
    static __device__ __forceinline__ type mul(type a, type b) { return __hmul2_rn(a, b); }
    static __device__ __forceinline__ type neg(type a) { return __hneg2(a); }
    static __device__ __forceinline__ type abs(type a) { return __habs2(a); }
    static __device__ __forceinline__ float2 unpack(type a) { return __bfloat1622float2(a); }
    static __device__ __forceinline__ type pack(float2 f) { return __float22bfloat162_rn(f); }
    static __device__ __forceinline__ type splat(float f) { return __float2bfloat162_rn(f); }
};

template <typename T, int OP>
__device__ __forceinline__ typename Pack2<T>::type apply_packed(typename Pack2<T>::type a, typename Pack2<T>::type b, float immf) {
    using PK = Pack2<T>;
    if constexpr (OP == TN_OP_ADD) return PK::add(a, b);
    else if constexpr (OP == TN_OP_SUB) return PK::sub(a, b);
    else if constexpr (OP == TN_OP_MUL) return PK::mul(a, b);
    else if constexpr (OP == TN_OP_NEG) return PK::neg(a);
    else if constexpr (OP == TN_OP_ABS) return PK::abs(a);
    else if constexpr (OP == TN_OP_SCALE) return PK::mul(a, PK::splat(immf));  // factor rounded to T first
    else if constexpr (stdx::is_same<T, __half>::value && (OP == TN_OP_LOG || OP == TN_OP_EXP)) {
        // A float16 value widened to float32 is never subnormal and a result below 2^-24 rounds
        // to zero in float16 anyway, so the flush-to-zero forms of the special-function unit
        // lose nothing and save the subnormal fix-up code around lg2 / ex2.
        const float2 x = PK::unpack(a);
        float2 r;
        if constexpr (OP == TN_OP_LOG) {
            asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(r.x) : "f"(x.x));
            asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(r.y) : "f"(x.y));
            r.x = __fmul_rn(r.x, 0.693147180559945309f);
            r.y = __fmul_rn(r.y, 0.693147180559945309f);
        } else {
            asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r.x) : "f"(__fmul_rn(x.x, 1.44269504088896341f)));
            asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r.y) : "f"(__fmul_rn(x.y, 1.44269504088896341f)));
        }
        return PK::pack(r);
    } else {
        const Imm imm{(double)immf, 0};
        const float2 x = PK::unpack(a), y = PK::unpack(b);
        float2 r;
        r.x = apply_op<OP, true, float>(x.x, y.x, imm);
        r.y = apply_op<OP, true, float>(x.y, y.y, imm);
        return PK::pack(r);
    }
}

template <typename T, typename P, int K, int V2, int VALUES>
__device__ __forceinline__ void eval_static_packed(typename Pack2<T>::type (&val)[VALUES][V2], const tn_eltwise_node_t* nodes) {
    static_assert(VALUES >= kMaxIn + P::N, "one value per input and node");
    if constexpr (K < P::N) {
        constexpr NodeSpec nd = P::nodes[K];
        const float immf = nodes[K].imm;
#pragma unroll
        for (int i = 0; i < V2; ++i) val[kMaxIn + K][i] = apply_packed<T, nd.op>(val[nd.lhs][i], val[nd.rhs][i], immf);
        eval_static_packed<T, P, K + 1, V2>(val, nodes);
    }
}

// One node on one 16-byte vector, opcode known at compile time. 16-bit types go through the packed
// path (same code as the compiled programs, so results are bit-identical to them); wider types
// compute per element and round on store.
template <typename T, int OP>
__device__ __forceinline__ Vec<T> node_on_vector(const Vec<T>& a, const Vec<T>& b, float immf) {
    Vec<T> r;
    if constexpr (sizeof(T) == 2) {
        using P2 = typename Pack2<T>::type;
#pragma unroll
        for (int i = 0; i < Vec<T>::N / 2; ++i)
            reinterpret_cast<P2*>(r.e)[i] = apply_packed<T, OP>(reinterpret_cast<const P2*>(a.e)[i], reinterpret_cast<const P2*>(b.e)[i], immf);
    } else {
        using C = typename compute_of<T>::type;
        const Imm imm{(double)immf, 0};
#pragma unroll
        for (int i = 0; i < Vec<T>::N; ++i)
            r.e[i] = from_compute<T, C>(round_to_storage<T, C>(apply_op<OP, false, C>(to_compute<C>(a.e[i]), to_compute<C>(b.e[i]), imm)));
    }
    return r;
}

// The interpreter's dispatch: one switch per node for all U vectors a thread holds, not per element.
template <typename T, int U>
__device__ __forceinline__ void node_dispatch(int op, const Vec<T> (&a)[U], const Vec<T> (&b)[U], float immf, Vec<T> (&r)[U]) {
#define TN_NODE_CASE(OP)                                                        \
    case OP:                                                                    \
        _Pragma("unroll") for (int u = 0; u < U; ++u) r[u] = node_on_vector<T, OP>(a[u], b[u], immf); \
        break;
    switch (op) {
        TN_NODE_CASE(TN_OP_ADD)
        TN_NODE_CASE(TN_OP_SUB)
        TN_NODE_CASE(TN_OP_MUL)
        TN_NODE_CASE(TN_OP_POW)
        TN_NODE_CASE(TN_OP_NEG)
        TN_NODE_CASE(TN_OP_LOG)
        TN_NODE_CASE(TN_OP_EXP)
        TN_NODE_CASE(TN_OP_SQRT)
        TN_NODE_CASE(TN_OP_RSQRT)
        TN_NODE_CASE(TN_OP_ABS)
        TN_NODE_CASE(TN_OP_SIN)
        TN_NODE_CASE(TN_OP_COS)
        TN_NODE_CASE(TN_OP_TAN)
        TN_NODE_CASE(TN_OP_SINH)
        TN_NODE_CASE(TN_OP_COSH)
        TN_NODE_CASE(TN_OP_TANH)
        TN_NODE_CASE(TN_OP_SCALE)
        default:
#pragma unroll
            for (int u = 0; u < U; ++u) r[u] = a[u];
            break;
    }
#undef TN_NODE_CASE
}

// The interpreter on U vectors at once. Every value (inputs, then one per node, rounded to the storage
// type like the node-by-node chain) lives in shared memory: 16 bytes per thread, vector and value,
// at word (value * U + u) * blockDim.x + thread. Nothing is shared between threads, so no barrier is
// needed; shared memory only stands in for a register file that can be indexed at run time.
// (Two alternatives measured slower on a six-node float16 expression over [8192,8192], 0.172 ms as
// written here: keeping the previous node's result in registers, with the host marking which operands
// and results can skip shared memory, 0.214 ms; a postfix program on a four-slot register stack with
// one switch case per (operation, slot), no shared memory at all, 0.253 ms.)
template <typename T, int U>
__device__ __forceinline__ void eval_interpreted(const Vec<T> (&vin)[U][kMaxIn], Vec<T> (&out)[U], const ProgArgs& g) {
    extern __shared__ uint4 program_values[];
    uint4* mine = program_values + threadIdx.x;
#pragma unroll
    for (int k = 0; k < kMaxIn; ++k)
        if (k < g.n_inputs) {
#pragma unroll
            for (int u = 0; u < U; ++u) mine[(k * U + u) * kThreads] = *reinterpret_cast<const uint4*>(&vin[u][k]);
        }
    for (int n = 0; n < g.n_nodes; ++n) {
        const tn_eltwise_node_t nd = g.nodes[n];
        Vec<T> a[U], b[U], r[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            *reinterpret_cast<uint4*>(&a[u]) = mine[(nd.lhs * U + u) * kThreads];
            *reinterpret_cast<uint4*>(&b[u]) = mine[(nd.rhs * U + u) * kThreads];
        }
        node_dispatch<T, U>(nd.opcode, a, b, nd.imm, r);
#pragma unroll
        for (int u = 0; u < U; ++u) mine[((kMaxIn + n) * U + u) * kThreads] = *reinterpret_cast<const uint4*>(&r[u]);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) *reinterpret_cast<uint4*>(&out[u]) = mine[((kMaxIn + g.n_nodes - 1) * U + u) * kThreads];
}

// Evaluates the program on one 16-byte vector of every input.
template <typename T, typename P>
__device__ __forceinline__ Vec<T> eval_vector(const Vec<T> (&vin)[kMaxIn], const ProgArgs& g) {
    using C = typename compute_of<T>::type;
    [[maybe_unused]] constexpr bool FAST = sizeof(T) == 2;
    constexpr int V = Vec<T>::N;
    constexpr bool STATIC = P::N > 0;
    Vec<T> out;
    if constexpr (STATIC && sizeof(T) == 2) {
        using P2 = typename Pack2<T>::type;
        constexpr int V2 = V / 2;
        P2 val[kMaxIn + P::N][V2];
#pragma unroll
        for (int k = 0; k < kMaxIn; ++k)
#pragma unroll
            for (int i = 0; i < V2; ++i)
                val[k][i] = k < g.n_inputs ? reinterpret_cast<const P2*>(vin[k].e)[i] : Pack2<T>::splat(0.0f);
        eval_static_packed<T, P, 0, V2>(val, g.nodes);
#pragma unroll
        for (int i = 0; i < V2; ++i) reinterpret_cast<P2*>(out.e)[i] = val[kMaxIn + P::N - 1][i];
    } else if constexpr (STATIC) {
        C val[kMaxIn + P::N][V];
#pragma unroll
        for (int k = 0; k < kMaxIn; ++k)
#pragma unroll
            for (int i = 0; i < V; ++i) val[k][i] = k < g.n_inputs ? to_compute<C>(vin[k].e[i]) : C(0);
        eval_static<T, P, 0, V>(val, g.nodes);
#pragma unroll
        for (int i = 0; i < V; ++i) out.e[i] = from_compute<T, C>(val[kMaxIn + P::N - 1][i]);
    } else {
        static_assert(STATIC, "interpreted programs go through eval_interpreted");
    }
    return out;
}

// A thread owns one 16-byte column slot and walks down the rows, UNROLL adjacent rows at a time.
// The loads of those rows are issued before any of them is consumed, so that enough bytes are in
// flight per SM to cover the HBM latency. A row-broadcast input has row pitch 0 and is simply
// re-read (from L1) every row; only when some input is column-broadcast (ANY_SCALAR) does the
// load path branch on the input kind.
template <typename T, typename P, int UNROLL, bool ANY_SCALAR>
__global__ void __launch_bounds__(kThreads) ew_program_rows(const __grid_constant__ ProgArgs g) {
    constexpr int V = Vec<T>::N;
    constexpr int NIN = P::NIN;
    const int64_t cvec = g.cols / V;
    const int64_t rstep = (int64_t)gridDim.y * UNROLL;
    for (int64_t cv = (int64_t)blockIdx.x * kThreads + threadIdx.x; cv < cvec; cv += (int64_t)gridDim.x * kThreads) {
        const int64_t c = cv * V;
        for (int64_t r0 = (int64_t)blockIdx.y * UNROLL; r0 < g.rows; r0 += rstep) {
            Vec<T> vin[UNROLL][kMaxIn];
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const int64_t r = r0 + u < g.rows ? r0 + u : g.rows - 1;  // the tail re-reads the last row
#pragma unroll
                for (int k = 0; k < NIN; ++k) {
                    if (P::N == 0 && k >= g.n_inputs) continue;
                    const T* base = static_cast<const T*>(g.in[k]);
                    if constexpr (ANY_SCALAR) {
                        if (g.inner[k]) vin[u][k] = load_vec(base + r * g.rs[k] + c);
                        else vin[u][k] = splat_vec(__ldg(base + r * g.rs[k]));
                    } else {
                        vin[u][k] = load_vec(base + r * g.rs[k] + c);
                    }
                }
            }
            if constexpr (P::N == 0) {
                Vec<T> outs[UNROLL];
                eval_interpreted<T, UNROLL>(vin, outs, g);
#pragma unroll
                for (int u = 0; u < UNROLL; ++u)
                    if (r0 + u < g.rows) store_vec(static_cast<T*>(g.d) + (r0 + u) * g.cols + c, outs[u]);
            } else {
#pragma unroll
                for (int u = 0; u < UNROLL; ++u)
                    if (r0 + u < g.rows) store_vec(static_cast<T*>(g.d) + (r0 + u) * g.cols + c, eval_vector<T, P>(vin[u], g));
            }
        }
    }
}


}  // namespace prog
}  // namespace tnb
