/*
 * TEST INFRASTRUCTURE — CPU restatement of the reference's algorithms for the operator hot path.
 *
 * This file is the parity oracle of the test-suite. It is never linked into, loaded by or called
 * from the product library (libtannic_b200.so); only tests/, the smoke check and the benchmark's
 * CPU-baseline leg may use it. Every function cites the reference code it restates
 * (paths relative to the reference project). Plain C, single-threaded scalar loops, soft
 * fp16/bf16 conversions, no FMA contraction (-ffp-contract=off), like the reference's own
 * `g++ -O2` build on x86-64.
 *
 * Parity pinning: tests/test_oracle_vs_reference.py checks this restatement bit-for-bit (integers,
 * indices, half add/sub/mul, accumulations) or to 1 ulp (libm calls) against the reference's own
 * CPU kernels compiled from its sources (oracle/_ref), against the golden vectors generated from
 * those kernels (tests/golden/*.npz) and against the literal vectors of the reference's test files.
 *
 * Accumulation modes (argument `acc`):
 *   ORC_ACC_STORAGE  accumulate in the result type exactly as the reference CPU kernels do
 *                    (src/cpu/matmul.cpp:32, src/cpu/conv2d.cpp:37, src/cpu/argred.cpp:32);
 *   ORC_ACC_WIDE     accumulate half types in float32 (float32 sums in float64, integers in
 *                    int64) — what the reference's own float-accumulating instantiations
 *                    (src/cpu/matmul.cpp:228, src/cpu/conv2d.cpp:232) and its device reductions
 *                    (src/cuda/argred.cu:167-187) do, and what the device backend implements.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#include "tannic_b200.h"

enum { ORC_ACC_STORAGE = 0, ORC_ACC_WIDE = 1 };

/* ------------------------------------------------------------------ half formats ------ */

static float bits_to_float(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static uint32_t float_to_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

/* IEEE binary16 -> float (exact). Host twin of the reference's soft float16_t,
 * src/types.cpp:6-60. */
static float half_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu;
    if (exp == 0) {
        if (man == 0) return bits_to_float(sign);
        float f = (float)man * 5.9604644775390625e-8f; /* 2^-24 */
        return sign ? -f : f;
    }
    if (exp == 31) return bits_to_float(sign | 0x7F800000u | (man << 13));
    return bits_to_float(sign | ((exp + 112u) << 23) | (man << 13));
}

/* float -> binary16, round to nearest even (what `std::float16_t(x)` does under GCC). */
static uint16_t float_to_half(float f) {
    uint32_t x = float_to_bits(f);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t ax = x & 0x7FFFFFFFu;
    if (ax >= 0x7F800000u) return (uint16_t)(sign | 0x7C00u | ((ax > 0x7F800000u) ? (0x200u | ((ax >> 13) & 0x3FFu)) : 0));
    if (ax >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u); /* rounds to >= 65520 -> inf */
    if (ax < 0x33000001u) return (uint16_t)sign;              /* <= 2^-25 -> 0 */
    int32_t e = (int32_t)(ax >> 23) - 127;
    uint32_t man = (ax & 0x7FFFFFu) | 0x800000u;
    int shift = (e < -14) ? (13 + (-14 - e)) : 13;
    uint32_t q = man >> shift, rem = man & ((1u << shift) - 1u), halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (q & 1u))) ++q;
    if (e < -14) return (uint16_t)(sign | q); /* subnormal (q may carry into the exponent: still right) */
    return (uint16_t)(sign | (((uint32_t)(e + 15) << 10) + (q - 0x400u)));
}

static float bf16_to_float(uint16_t h) { return bits_to_float((uint32_t)h << 16); }

/* float -> bfloat16, round to nearest even (`std::bfloat16_t(x)` under GCC; note that the
 * reference's own soft bfloat16_t truncates instead, src/types.cpp:74-78 — kernels use the
 * compiler type, so RNE is what they see). */
static uint16_t float_to_bf16(float f) {
    uint32_t x = float_to_bits(f);
    if ((x & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((x >> 16) | 0x40u);
    uint32_t lsb = (x >> 16) & 1u;
    x += 0x7FFFu + lsb;
    return (uint16_t)(x >> 16);
}

/* double -> half types: GCC converts double -> _Float16 / __bf16 with a single rounding. */
static uint16_t double_to_half(double d) {
    float f = (float)d;
    /* guard against double rounding: if the float conversion was inexact and landed on a half
     * tie, nudge toward the true value */
    if ((double)f != d && isfinite(f)) {
        uint32_t b = float_to_bits(f);
        if ((b & 0x1FFFu) == 0x1000u) b += ((double)f < d) == !(b >> 31) ? 1u : (uint32_t)-1;
        f = bits_to_float(b);
    }
    return float_to_half(f);
}
static uint16_t double_to_bf16(double d) {
    float f = (float)d;
    if ((double)f != d && isfinite(f)) {
        uint32_t b = float_to_bits(f);
        if ((b & 0xFFFFu) == 0x8000u) b += ((double)f < d) == !(b >> 31) ? 1u : (uint32_t)-1;
        f = bits_to_float(b);
    }
    return float_to_bf16(f);
}

/* Exposed for the tests (seeded input generation uses the same conversions). */
uint16_t orc_float_to_half(float f) { return float_to_half(f); }
uint16_t orc_float_to_bf16(float f) { return float_to_bf16(f); }
float orc_half_to_float(uint16_t h) { return half_to_float(h); }
float orc_bf16_to_float(uint16_t h) { return bf16_to_float(h); }

/* ------------------------------------------------------------------ typed access ------ */

static int is_int(int dt) { return dt >= TN_INT8 && dt <= TN_INT64; }
static int is_half(int dt) { return dt == TN_FLOAT16 || dt == TN_BFLOAT16; }
static int is_float(int dt) { return dt >= TN_FLOAT16 && dt <= TN_FLOAT64; }
static int is_numeric(int dt) { return dt >= TN_INT8 && dt <= TN_FLOAT64; }

static double load_f64(const void* p, int dt, int64_t i) {
    switch (dt) {
        case TN_INT8: return (double)((const int8_t*)p)[i];
        case TN_INT16: return (double)((const int16_t*)p)[i];
        case TN_INT32: return (double)((const int32_t*)p)[i];
        case TN_INT64: return (double)((const int64_t*)p)[i];
        case TN_FLOAT16: return (double)half_to_float(((const uint16_t*)p)[i]);
        case TN_BFLOAT16: return (double)bf16_to_float(((const uint16_t*)p)[i]);
        case TN_FLOAT32: return (double)((const float*)p)[i];
        case TN_FLOAT64: return ((const double*)p)[i];
        default: return 0.0;
    }
}
static float load_f32(const void* p, int dt, int64_t i) {
    switch (dt) {
        case TN_INT8: return (float)((const int8_t*)p)[i];
        case TN_INT16: return (float)((const int16_t*)p)[i];
        case TN_INT32: return (float)((const int32_t*)p)[i];
        case TN_INT64: return (float)((const int64_t*)p)[i];
        case TN_FLOAT16: return half_to_float(((const uint16_t*)p)[i]);
        case TN_BFLOAT16: return bf16_to_float(((const uint16_t*)p)[i]);
        case TN_FLOAT32: return ((const float*)p)[i];
        case TN_FLOAT64: return (float)((const double*)p)[i];
        default: return 0.0f;
    }
}
static int64_t load_i64(const void* p, int dt, int64_t i) {
    switch (dt) {
        case TN_INT8: return ((const int8_t*)p)[i];
        case TN_INT16: return ((const int16_t*)p)[i];
        case TN_INT32: return ((const int32_t*)p)[i];
        case TN_INT64: return ((const int64_t*)p)[i];
        default: return 0;
    }
}
static void store_f64(void* p, int dt, int64_t i, double v) {
    switch (dt) {
        case TN_INT8: ((int8_t*)p)[i] = (int8_t)(int64_t)v; break;
        case TN_INT16: ((int16_t*)p)[i] = (int16_t)(int64_t)v; break;
        case TN_INT32: ((int32_t*)p)[i] = (int32_t)(int64_t)v; break;
        case TN_INT64: ((int64_t*)p)[i] = (int64_t)v; break;
        case TN_FLOAT16: ((uint16_t*)p)[i] = double_to_half(v); break;
        case TN_BFLOAT16: ((uint16_t*)p)[i] = double_to_bf16(v); break;
        case TN_FLOAT32: ((float*)p)[i] = (float)v; break;
        case TN_FLOAT64: ((double*)p)[i] = v; break;
        default: break;
    }
}
static void store_f32(void* p, int dt, int64_t i, float v) {
    switch (dt) {
        case TN_FLOAT16: ((uint16_t*)p)[i] = float_to_half(v); break;
        case TN_BFLOAT16: ((uint16_t*)p)[i] = float_to_bf16(v); break;
        case TN_FLOAT32: ((float*)p)[i] = v; break;
        default: store_f64(p, dt, i, (double)v); break;
    }
}
static void store_i64(void* p, int dt, int64_t i, int64_t v) {
    switch (dt) {
        case TN_INT8: ((int8_t*)p)[i] = (int8_t)v; break;
        case TN_INT16: ((int16_t*)p)[i] = (int16_t)v; break;
        case TN_INT32: ((int32_t*)p)[i] = (int32_t)v; break;
        case TN_INT64: ((int64_t*)p)[i] = v; break;
        default: store_f64(p, dt, i, (double)v); break;
    }
}

/* Rounds a float to the precision of storage dtype `dt` and back (identity for f32). */
static float round_through(float v, int dt) {
    if (dt == TN_FLOAT16) return half_to_float(float_to_half(v));
    if (dt == TN_BFLOAT16) return bf16_to_float(float_to_bf16(v));
    return v;
}

/* Arithmetic class of an operand pair: 0 = integer (wrapping), 1 = float32, 2 = float64.
 * Mirrors the result types of the dispatch tables in src/cpu/ops-binary.cpp:168-430 and
 * src/cpu/matmul.cpp:189-252. */
static int compute_class(int a, int b) {
    if (a == TN_FLOAT64 || b == TN_FLOAT64) return 2;
    if ((is_float(a) && b == TN_INT64) || (is_float(b) && a == TN_INT64)) return 2;
    if (is_float(a) || is_float(b)) return 1;
    return 0;
}

static int half_partner_ok(int h, int o) { return o == h || o == TN_FLOAT32 || o == TN_FLOAT64 || is_int(o); }
static int wide_ok(int o) { return o == TN_FLOAT32 || o == TN_FLOAT64 || o == TN_INT32; }

/* Supported operand pairs: src/cpu/ops-binary.cpp:168-430 (pow has no integer entries). */
static int pair_supported(int a, int b, int allow_int_pair) {
    if (!is_numeric(a) || !is_numeric(b)) return 0;
    if (is_int(a) && is_int(b)) return allow_int_pair;
    if (is_half(a)) return half_partner_ok(a, b);
    if (is_half(b)) return half_partner_ok(b, a);
    return wide_ok(a) && wide_ok(b);
}

/* ------------------------------------------------------------------ elementwise ------- */

enum { ORC_ADD = 0, ORC_SUB, ORC_MUL, ORC_POW };

/* src/cpu/ops-binary.cpp:65-128 (launchBinaryOpKernel): operands are aligned to the result's
 * rank from the right, extent-1 dims read with stride 0, the result is written through its
 * own strides; functors at :130-160. */
tn_status orc_binary(int op, const tn_tensor_t* a, const tn_tensor_t* b, tn_tensor_t* d) {
    if (!pair_supported(a->dtype, b->dtype, op != ORC_POW) || !is_numeric(d->dtype)) return TN_UNSUPPORTED_DTYPE;
    const int rank = d->rank, off0 = rank - a->rank, off1 = rank - b->rank;
    int64_t s0[TN_MAX_RANK] = {0}, s1[TN_MAX_RANK] = {0};
    for (int dim = 0; dim < rank; ++dim) {
        size_t z0 = dim >= off0 ? a->shape.sizes[dim - off0] : 1, z1 = dim >= off1 ? b->shape.sizes[dim - off1] : 1;
        s0[dim] = z0 == 1 ? 0 : a->strides.sizes[dim - off0];
        s1[dim] = z1 == 1 ? 0 : b->strides.sizes[dim - off1];
    }
    const int cls = compute_class(a->dtype, b->dtype);
    const int same_half = a->dtype == b->dtype && is_half(a->dtype);
    for (size_t lin = 0; lin < d->size; ++lin) {
        int64_t o0 = 0, o1 = 0, od = 0;
        size_t rem = lin;
        for (int dim = rank - 1; dim >= 0; --dim) {
            size_t c = rem % d->shape.sizes[dim];
            rem /= d->shape.sizes[dim];
            o0 += (int64_t)c * s0[dim];
            o1 += (int64_t)c * s1[dim];
            od += (int64_t)c * d->strides.sizes[dim];
        }
        if (cls == 0) {
            uint64_t x = (uint64_t)load_i64(a->address, a->dtype, o0), y = (uint64_t)load_i64(b->address, b->dtype, o1);
            uint64_t r = op == ORC_ADD ? x + y : op == ORC_SUB ? x - y : x * y;
            store_i64(d->address, d->dtype, od, (int64_t)r);
        } else if (cls == 1) {
            float x = load_f32(a->address, a->dtype, o0), y = load_f32(b->address, b->dtype, o1);
            float r = op == ORC_ADD ? x + y : op == ORC_SUB ? x - y : op == ORC_MUL ? x * y : powf(x, y);
            /* half (op) half yields a half in the reference, even where the table stores it wider */
            if (same_half) r = round_through(r, a->dtype);
            store_f32(d->address, d->dtype, od, r);
        } else {
            double x = load_f64(a->address, a->dtype, o0), y = load_f64(b->address, b->dtype, o1);
            double r = op == ORC_ADD ? x + y : op == ORC_SUB ? x - y : op == ORC_MUL ? x * y : pow(x, y);
            store_f64(d->address, d->dtype, od, r);
        }
    }
    return TN_SUCCESS;
}

enum {
    ORC_NEG = 0, ORC_REPACK, ORC_LOG, ORC_EXP, ORC_SQRT, ORC_RSQRT, ORC_ABS, ORC_SIN, ORC_COS, ORC_TAN,
    ORC_SINH, ORC_COSH, ORC_TANH
};

static float unary_f32(int op, float x) {
    switch (op) {
        case ORC_NEG: return -x;
        case ORC_LOG: return logf(x);
        case ORC_EXP: return expf(x);
        case ORC_SQRT: return sqrtf(x);
        case ORC_ABS: return fabsf(x);
        case ORC_SIN: return sinf(x);
        case ORC_COS: return cosf(x);
        case ORC_TAN: return tanf(x);
        case ORC_SINH: return sinhf(x);
        case ORC_COSH: return coshf(x);
        case ORC_TANH: return tanhf(x);
        default: return x;
    }
}
static double unary_f64(int op, double x) {
    switch (op) {
        case ORC_NEG: return -x;
        case ORC_LOG: return log(x);
        case ORC_EXP: return exp(x);
        case ORC_SQRT: return sqrt(x);
        case ORC_ABS: return fabs(x);
        case ORC_SIN: return sin(x);
        case ORC_COS: return cos(x);
        case ORC_TAN: return tan(x);
        case ORC_SINH: return sinh(x);
        case ORC_COSH: return cosh(x);
        case ORC_TANH: return tanh(x);
        default: return x;
    }
}

/* src/cpu/ops-unary.cpp:20-118 (kernels: the source may be strided and is read with the
 * result's extents, the result is written densely) and :120-200 (functors; Rsqrt is
 * `1.0 / std::sqrt(a + eps)` in double), dtype switches at :202-370. */
tn_status orc_unary(int op, const tn_tensor_t* x, tn_tensor_t* d, float eps) {
    const int dt = x->dtype;
    if (op == ORC_NEG || op == ORC_REPACK) { if (!is_numeric(dt)) return TN_UNSUPPORTED_DTYPE; }
    else if (op == ORC_ABS) { if (!(is_float(dt) || dt == TN_INT32 || dt == TN_INT64)) return TN_UNSUPPORTED_DTYPE; }
    else if (!is_float(dt)) return TN_UNSUPPORTED_DTYPE;
    size_t cnt[TN_MAX_RANK] = {0};
    const int rank = x->rank;
    for (size_t idx = 0; idx < d->size; ++idx) {
        int64_t off = 0;
        for (int dim = 0; dim < rank; ++dim) off += (int64_t)(d->shape.sizes[dim] == 1 ? 0 : cnt[dim]) * x->strides.sizes[dim];
        if (is_int(dt)) {
            int64_t v = load_i64(x->address, dt, off);
            uint64_t u = (uint64_t)v;
            if (op == ORC_NEG) v = (int64_t)(0 - u);
            else if (op == ORC_ABS) v = v < 0 ? (int64_t)(0 - u) : v;
            store_i64(d->address, d->dtype, (int64_t)idx, v);
        } else if (op == ORC_RSQRT) {
            store_f64(d->address, d->dtype, (int64_t)idx, 1.0 / sqrt(load_f64(x->address, dt, off) + (double)eps));
        } else if (dt == TN_FLOAT64) {
            store_f64(d->address, d->dtype, (int64_t)idx, unary_f64(op, load_f64(x->address, dt, off)));
        } else {
            /* std::log(std::float16_t) etc. evaluate the float32 function and narrow */
            store_f32(d->address, d->dtype, (int64_t)idx, unary_f32(op, load_f32(x->address, dt, off)));
        }
        for (int dim = rank - 1; dim >= 0; --dim) {
            if (++cnt[dim] < d->shape.sizes[dim]) break;
            cnt[dim] = 0;
        }
    }
    return TN_SUCCESS;
}

/* src/cpu/ops-scale.cpp:15-122: dst = src * scalar, same dtype only; integer entries use the
 * unsigned types, i.e. wrap. */
tn_status orc_scale(const tn_tensor_t* x, const tn_scalar_t* sc, tn_tensor_t* d) {
    const int dt = x->dtype;
    if (sc->dtype != dt || !is_numeric(dt)) return TN_UNSUPPORTED_DTYPE;
    size_t cnt[TN_MAX_RANK] = {0};
    const int rank = x->rank;
    for (size_t idx = 0; idx < d->size; ++idx) {
        int64_t off = 0;
        for (int dim = 0; dim < rank; ++dim) off += (int64_t)(d->shape.sizes[dim] == 1 ? 0 : cnt[dim]) * x->strides.sizes[dim];
        if (is_int(dt)) {
            uint64_t r = (uint64_t)load_i64(x->address, dt, off) * (uint64_t)load_i64(sc->address, dt, 0);
            store_i64(d->address, d->dtype, (int64_t)idx, (int64_t)r);
        } else if (dt == TN_FLOAT64) {
            store_f64(d->address, d->dtype, (int64_t)idx, load_f64(x->address, dt, off) * load_f64(sc->address, dt, 0));
        } else {
            store_f32(d->address, d->dtype, (int64_t)idx, load_f32(x->address, dt, off) * load_f32(sc->address, dt, 0));
        }
        for (int dim = rank - 1; dim >= 0; --dim) {
            if (++cnt[dim] < d->shape.sizes[dim]) break;
            cnt[dim] = 0;
        }
    }
    return TN_SUCCESS;
}

/* ------------------------------------------------------------------ matmul ------------ */

/* src/cpu/matmul.cpp:21-41 (gemmKernel: i, j, then k ascending; `sum += D(a) * D(b)`),
 * :43-50 (isTransposed: stride[-1] > stride[-2]; the leading dimension is the larger stride and
 * the other one is taken to be 1), :96-124 (computeOffsets: batch index decoded over the
 * result's batch dims, extent-1 or missing operand dims contribute offset 0) and :126-176.
 *
 * `wrap_batch_u8` != 0 reproduces the reference's defect of passing the batch counter through a
 * uint8_t parameter (src/cpu/matmul.cpp:101,146-148): batches >= 256 alias batches 0..255.
 * The device backend does not reproduce it; the flag exists for the regression test. */
tn_status orc_gemm(const tn_tensor_t* a, const tn_tensor_t* b, tn_tensor_t* d, int acc, int wrap_batch_u8) {
    if (!pair_supported(a->dtype, b->dtype, 1) || !is_numeric(d->dtype)) return TN_UNSUPPORTED_DTYPE;
    if (a->rank < 2 || b->rank < 2 || d->rank < 2) return TN_ERROR;
    const int ra = a->rank, rb = b->rank, rd = d->rank;
    const int64_t M = (int64_t)d->shape.sizes[rd - 2], N = (int64_t)d->shape.sizes[rd - 1], K = (int64_t)a->shape.sizes[ra - 1];
    const int a_trans = a->strides.sizes[ra - 1] > a->strides.sizes[ra - 2];
    const int b_trans = b->strides.sizes[rb - 1] > b->strides.sizes[rb - 2];
    const int64_t a_ld = a_trans ? a->strides.sizes[ra - 1] : a->strides.sizes[ra - 2];
    const int64_t b_ld = b_trans ? b->strides.sizes[rb - 1] : b->strides.sizes[rb - 2];
    const int64_t d_ld = d->strides.sizes[rd - 2];
    const int batch_rank = rd - 2;
    int64_t batches = 1;
    for (int dim = 0; dim < batch_rank; ++dim) batches *= (int64_t)d->shape.sizes[dim];
    const int cls = compute_class(a->dtype, b->dtype);
    /* the reference accumulates in the table's D type: half for half x half */
    const int half_acc = acc == ORC_ACC_STORAGE && a->dtype == b->dtype && is_half(a->dtype);
    for (int64_t batch = 0; batch < batches; ++batch) {
        int64_t oa = 0, ob = 0, od = 0;
        int64_t rem = wrap_batch_u8 ? (int64_t)(uint8_t)batch : batch;
        int64_t idx[TN_MAX_RANK] = {0};
        for (int dim = batch_rank - 1; dim >= 0; --dim) {
            idx[dim] = rem % (int64_t)d->shape.sizes[dim];
            rem /= (int64_t)d->shape.sizes[dim];
        }
        for (int dim = 0; dim < batch_rank; ++dim) {
            const int da = dim + (ra - rd), db = dim + (rb - rd);
            if (da >= 0 && a->shape.sizes[da] != 1) oa += idx[dim] * a->strides.sizes[da];
            if (db >= 0 && b->shape.sizes[db] != 1) ob += idx[dim] * b->strides.sizes[db];
            od += idx[dim] * d->strides.sizes[dim];
        }
        for (int64_t i = 0; i < M; ++i) {
            for (int64_t j = 0; j < N; ++j) {
                const int64_t c_off = od + i * d_ld + j;
                if (cls == 0) {
                    uint64_t sum = 0;
                    for (int64_t k = 0; k < K; ++k) {
                        const int64_t ai = oa + (a_trans ? k * a_ld + i : i * a_ld + k), bi = ob + (b_trans ? j * b_ld + k : k * b_ld + j);
                        sum += (uint64_t)load_i64(a->address, a->dtype, ai) * (uint64_t)load_i64(b->address, b->dtype, bi);
                    }
                    store_i64(d->address, d->dtype, c_off, (int64_t)sum);
                } else if (cls == 1) {
                    float sum = 0.0f;
                    for (int64_t k = 0; k < K; ++k) {
                        const int64_t ai = oa + (a_trans ? k * a_ld + i : i * a_ld + k), bi = ob + (b_trans ? j * b_ld + k : k * b_ld + j);
                        const float prod = load_f32(a->address, a->dtype, ai) * load_f32(b->address, b->dtype, bi);
                        sum = sum + prod;
                        if (half_acc) sum = round_through(sum, a->dtype);
                    }
                    store_f32(d->address, d->dtype, c_off, sum);
                } else {
                    double sum = 0.0;
                    for (int64_t k = 0; k < K; ++k) {
                        const int64_t ai = oa + (a_trans ? k * a_ld + i : i * a_ld + k), bi = ob + (b_trans ? j * b_ld + k : k * b_ld + j);
                        sum += load_f64(a->address, a->dtype, ai) * load_f64(b->address, b->dtype, bi);
                    }
                    store_f64(d->address, d->dtype, c_off, sum);
                }
            }
        }
    }
    return TN_SUCCESS;
}

/* ------------------------------------------------------------------ conv2d ------------ */

/* src/cpu/conv2d.cpp:17-64 (conv2dKernel: n, co, oh, ow, then ci, kh, kw ascending with
 * out-of-range taps skipped), :66-113 (bias seeds the accumulator), :116-197 (rank / shape
 * checks -> ERROR, floor output extent), :221-253 (equal dtypes only). `bias` may be NULL. */
tn_status orc_conv2d(const tn_tensor_t* x, const tn_tensor_t* w, const tn_tensor_t* bias, tn_tensor_t* y,
                     const size_t pad[2], const size_t stride[2], int acc) {
    if (x->dtype != w->dtype || !is_numeric(x->dtype)) return TN_UNSUPPORTED_DTYPE;
    if (x->rank != 4 || w->rank != 4 || y->rank != 4 || (bias && bias->rank != 1)) return TN_ERROR;
    const int dt = x->dtype;
    const int64_t N = (int64_t)x->shape.sizes[0], Cin = (int64_t)x->shape.sizes[1], H = (int64_t)x->shape.sizes[2], W = (int64_t)x->shape.sizes[3];
    const int64_t Cout = (int64_t)w->shape.sizes[0], Kh = (int64_t)w->shape.sizes[2], Kw = (int64_t)w->shape.sizes[3];
    if ((int64_t)w->shape.sizes[1] != Cin || (bias && (int64_t)bias->shape.sizes[0] != Cout)) return TN_ERROR;
    const int64_t Ho = (H + 2 * (int64_t)pad[0] - Kh) / (int64_t)stride[0] + 1, Wo = (W + 2 * (int64_t)pad[1] - Kw) / (int64_t)stride[1] + 1;
    if ((int64_t)y->shape.sizes[0] != N || (int64_t)y->shape.sizes[1] != Cout || (int64_t)y->shape.sizes[2] != Ho || (int64_t)y->shape.sizes[3] != Wo) return TN_ERROR;
    const int64_t* xs = x->strides.sizes; const int64_t* ws = w->strides.sizes; const int64_t* ys = y->strides.sizes;
    const int half_acc = acc == ORC_ACC_STORAGE && is_half(dt);
    for (int64_t n = 0; n < N; ++n)
    for (int64_t co = 0; co < Cout; ++co)
    for (int64_t oh = 0; oh < Ho; ++oh)
    for (int64_t ow = 0; ow < Wo; ++ow) {
        const int64_t bh = oh * (int64_t)stride[0] - (int64_t)pad[0], bw = ow * (int64_t)stride[1] - (int64_t)pad[1];
        const int64_t yo = n * ys[0] + co * ys[1] + oh * ys[2] + ow * ys[3];
        if (is_int(dt)) {
            uint64_t sum = bias ? (uint64_t)load_i64(bias->address, dt, co * bias->strides.sizes[0]) : 0;
            for (int64_t ci = 0; ci < Cin; ++ci) for (int64_t kh = 0; kh < Kh; ++kh) {
                const int64_t ih = bh + kh; if (ih < 0 || ih >= H) continue;
                for (int64_t kw = 0; kw < Kw; ++kw) {
                    const int64_t iw = bw + kw; if (iw < 0 || iw >= W) continue;
                    sum += (uint64_t)load_i64(x->address, dt, n * xs[0] + ci * xs[1] + ih * xs[2] + iw * xs[3]) *
                           (uint64_t)load_i64(w->address, dt, co * ws[0] + ci * ws[1] + kh * ws[2] + kw * ws[3]);
                }
            }
            store_i64(y->address, dt, yo, (int64_t)sum);
        } else if (dt == TN_FLOAT64) {
            double sum = bias ? load_f64(bias->address, dt, co * bias->strides.sizes[0]) : 0.0;
            for (int64_t ci = 0; ci < Cin; ++ci) for (int64_t kh = 0; kh < Kh; ++kh) {
                const int64_t ih = bh + kh; if (ih < 0 || ih >= H) continue;
                for (int64_t kw = 0; kw < Kw; ++kw) {
                    const int64_t iw = bw + kw; if (iw < 0 || iw >= W) continue;
                    sum += load_f64(x->address, dt, n * xs[0] + ci * xs[1] + ih * xs[2] + iw * xs[3]) *
                           load_f64(w->address, dt, co * ws[0] + ci * ws[1] + kh * ws[2] + kw * ws[3]);
                }
            }
            store_f64(y->address, dt, yo, sum);
        } else {
            float sum = bias ? load_f32(bias->address, dt, co * bias->strides.sizes[0]) : 0.0f;
            for (int64_t ci = 0; ci < Cin; ++ci) for (int64_t kh = 0; kh < Kh; ++kh) {
                const int64_t ih = bh + kh; if (ih < 0 || ih >= H) continue;
                for (int64_t kw = 0; kw < Kw; ++kw) {
                    const int64_t iw = bw + kw; if (iw < 0 || iw >= W) continue;
                    const float prod = load_f32(x->address, dt, n * xs[0] + ci * xs[1] + ih * xs[2] + iw * xs[3]) *
                                       load_f32(w->address, dt, co * ws[0] + ci * ws[1] + kh * ws[2] + kw * ws[3]);
                    sum = sum + prod;
                    if (half_acc) sum = round_through(sum, dt);
                }
            }
            store_f32(y->address, dt, yo, sum);
        }
    }
    return TN_SUCCESS;
}

/* ------------------------------------------------------------------ reductions -------- */

enum { ORC_ARGMAX = 0, ORC_ARGMIN, ORC_SUM, ORC_MEAN, ORC_MAX };

/* src/cpu/argred.cpp:19-77 (sum / mean: accumulate over the axis in ascending order, mean
 * divides by the count in the accumulator type), :80-147 (argmax / argmin: strict comparison
 * against an initial -inf / +inf or integer limit with index 0, ties keep the lower index,
 * NaN is never selected), :183-285 (outputs in logical order of the remaining dims),
 * :289-347 (dtypes: sum for all numeric types, mean for floats only, indices are int64).
 * ORC_MAX has no reference counterpart: it is the value at the argmax index. */
tn_status orc_reduce(int kind, const tn_tensor_t* x, tn_tensor_t* d, uint8_t axis, int acc) {
    const int dt = x->dtype, rank = x->rank;
    if (axis >= rank) return TN_ERROR;
    if (kind == ORC_MEAN ? !is_float(dt) : !is_numeric(dt)) return TN_UNSUPPORTED_DTYPE;
    const int64_t len = (int64_t)x->shape.sizes[axis], ax_stride = x->strides.sizes[axis];
    size_t total = 1;
    for (int dim = 0; dim < rank; ++dim) if (dim != axis) total *= x->shape.sizes[dim];
    size_t cnt[TN_MAX_RANK] = {0};
    for (size_t o = 0; o < total; ++o) {
        int64_t base = 0;
        for (int dim = 0; dim < rank; ++dim) if (dim != axis) base += (int64_t)cnt[dim] * x->strides.sizes[dim];
        if (kind == ORC_SUM || kind == ORC_MEAN) {
            if (is_int(dt)) {
                uint64_t sum = 0;
                for (int64_t i = 0; i < len; ++i) sum += (uint64_t)load_i64(x->address, dt, base + i * ax_stride);
                store_i64(d->address, d->dtype, (int64_t)o, (int64_t)sum);
            } else if (dt == TN_FLOAT64 || (dt == TN_FLOAT32 && acc == ORC_ACC_WIDE)) {
                double sum = 0.0;
                for (int64_t i = 0; i < len; ++i) sum += load_f64(x->address, dt, base + i * ax_stride);
                if (kind == ORC_MEAN) sum = sum / (double)len;
                store_f64(d->address, d->dtype, (int64_t)o, sum);
            } else {
                float sum = 0.0f;
                const int narrow = acc == ORC_ACC_STORAGE && is_half(dt);
                for (int64_t i = 0; i < len; ++i) {
                    sum = sum + load_f32(x->address, dt, base + i * ax_stride);
                    if (narrow) sum = round_through(sum, dt);
                }
                if (kind == ORC_MEAN) {
                    sum = sum / (narrow ? round_through((float)len, dt) : (float)len);
                }
                store_f32(d->address, d->dtype, (int64_t)o, sum);
            }
        } else {
            const int minimise = kind == ORC_ARGMIN;
            int64_t best = 0;
            if (is_int(dt)) {
                int64_t lo = dt == TN_INT8 ? INT8_MIN : dt == TN_INT16 ? INT16_MIN : dt == TN_INT32 ? INT32_MIN : INT64_MIN;
                int64_t hi = dt == TN_INT8 ? INT8_MAX : dt == TN_INT16 ? INT16_MAX : dt == TN_INT32 ? INT32_MAX : INT64_MAX;
                int64_t bv = minimise ? hi : lo;
                for (int64_t i = 0; i < len; ++i) {
                    const int64_t v = load_i64(x->address, dt, base + i * ax_stride);
                    if ((minimise ? v < bv : v > bv) || (v == bv && i < best)) { bv = v; best = i; }
                }
            } else {
                double bv = minimise ? INFINITY : -INFINITY;
                for (int64_t i = 0; i < len; ++i) {
                    const double v = load_f64(x->address, dt, base + i * ax_stride);
                    if ((minimise ? v < bv : v > bv) || (v == bv && i < best)) { bv = v; best = i; }
                }
            }
            if (kind == ORC_MAX) {
                if (is_int(dt)) store_i64(d->address, d->dtype, (int64_t)o, len > 0 ? load_i64(x->address, dt, base + best * ax_stride) : 0);
                else store_f64(d->address, d->dtype, (int64_t)o, len > 0 ? load_f64(x->address, dt, base + best * ax_stride) : 0.0);
            } else {
                ((int64_t*)d->address)[o] = best;
            }
        }
        for (int dim = rank - 1; dim >= 0; --dim) {
            if (dim == axis) continue;
            if (++cnt[dim] < x->shape.sizes[dim]) break;
            cnt[dim] = 0;
        }
    }
    return TN_SUCCESS;
}

/* ------------------------------------------------------------------ utilities --------- */

/* src/cpu/cpy.cpp:19-43: element copy between two strided views of one logical shape;
 * extent-1 dims of either side stay at offset 0. */
static size_t dtype_bytes(int dt) {
    switch (dt) {
        case TN_BOOLEAN: case TN_INT8: return 1;
        case TN_INT16: case TN_FLOAT16: case TN_BFLOAT16: return 2;
        case TN_INT32: case TN_FLOAT32: return 4;
        case TN_INT64: case TN_FLOAT64: case TN_COMPLEX64: return 8;
        case TN_COMPLEX128: return 16;
        default: return 0;
    }
}

tn_status orc_cpy(const tn_tensor_t* s, tn_tensor_t* d) {
    const size_t esize = dtype_bytes((int)s->dtype);
    if (s->dtype != d->dtype || esize == 0) return TN_UNSUPPORTED_DTYPE;
    const int rank = s->rank;
    size_t cnt[TN_MAX_RANK] = {0};
    for (size_t idx = 0; idx < s->size; ++idx) {
        int64_t so = 0, dof = 0;
        for (int dim = 0; dim < rank; ++dim) {
            so += (int64_t)(s->shape.sizes[dim] == 1 ? 0 : cnt[dim]) * s->strides.sizes[dim];
            dof += (int64_t)(d->shape.sizes[dim] == 1 ? 0 : cnt[dim]) * d->strides.sizes[dim];
        }
        memcpy((char*)d->address + dof * (int64_t)esize, (const char*)s->address + so * (int64_t)esize, esize);
        for (int dim = rank - 1; dim >= 0; --dim) {
            if (++cnt[dim] < d->shape.sizes[dim]) break;
            cnt[dim] = 0;
        }
    }
    return TN_SUCCESS;
}

/* src/cpu/val.cpp:17-70: every element must satisfy |a - b| <= atol + rtol * |b| (evaluated in
 * double; a NaN never fails the test). Floating dtypes only. */
tn_status orc_allclose(const tn_tensor_t* a, const tn_tensor_t* b, double rtol, double atol, int* close) {
    if (a->dtype != b->dtype || !is_float(a->dtype)) return TN_UNSUPPORTED_DTYPE;
    const int rank = a->rank;
    size_t cnt[TN_MAX_RANK] = {0};
    *close = 1;
    for (size_t idx = 0; idx < a->size; ++idx) {
        int64_t oa = 0, ob = 0;
        for (int dim = 0; dim < rank; ++dim) {
            oa += (int64_t)cnt[dim] * a->strides.sizes[dim];
            ob += (int64_t)cnt[dim] * b->strides.sizes[dim];
        }
        const double x = load_f64(a->address, a->dtype, oa), y = load_f64(b->address, b->dtype, ob);
        if (fabs(x - y) > atol + rtol * fabs(y)) { *close = 0; return TN_SUCCESS; }
        for (int dim = rank - 1; dim >= 0; --dim) {
            if (++cnt[dim] < a->shape.sizes[dim]) break;
            cnt[dim] = 0;
        }
    }
    return TN_SUCCESS;
}

/* src/cpu/cmps.cpp:16-41 and :96-118: operands of one dtype walked with their own strides over the
 * result's shape; the result is boolean, bit-packed: the (size + 7) / 8 bytes are cleared, then
 * element i sets bit i % 8 of byte i / 8. op: 0 eq, 1 ne, 2 gt, 3 ge, 4 lt, 5 le. Integers compare
 * as int64, floats as double (exact for every storage type); an extent-1 operand dimension reads
 * offset 0. */
tn_status orc_compare(int op, const tn_tensor_t* a, const tn_tensor_t* b, tn_tensor_t* d) {
    if (a->dtype != b->dtype || !is_numeric((int)a->dtype) || d->dtype != TN_BOOLEAN) return TN_UNSUPPORTED_DTYPE;
    if (op < 0 || op > 5) return TN_ERROR;
    const int rank = d->rank;
    uint8_t* out = (uint8_t*)d->address;
    memset(out, 0, (d->size + 7) / 8);
    size_t cnt[TN_MAX_RANK] = {0};
    for (size_t idx = 0; idx < d->size; ++idx) {
        int64_t oa = 0, ob = 0;
        for (int dim = 0; dim < rank; ++dim) {
            oa += (int64_t)(a->shape.sizes[dim] == 1 ? 0 : cnt[dim]) * a->strides.sizes[dim];
            ob += (int64_t)(b->shape.sizes[dim] == 1 ? 0 : cnt[dim]) * b->strides.sizes[dim];
        }
        int r;
        if (is_int((int)a->dtype)) {
            const int64_t x = load_i64(a->address, (int)a->dtype, oa), y = load_i64(b->address, (int)b->dtype, ob);
            r = op == 0 ? x == y : op == 1 ? x != y : op == 2 ? x > y : op == 3 ? x >= y : op == 4 ? x < y : x <= y;
        } else {
            const double x = load_f64(a->address, (int)a->dtype, oa), y = load_f64(b->address, (int)b->dtype, ob);
            r = op == 0 ? x == y : op == 1 ? x != y : op == 2 ? x > y : op == 3 ? x >= y : op == 4 ? x < y : x <= y;
        }
        out[idx / 8] |= (uint8_t)((r ? 1u : 0u) << (idx % 8));
        for (int dim = rank - 1; dim >= 0; --dim) {
            if (++cnt[dim] < d->shape.sizes[dim]) break;
            cnt[dim] = 0;
        }
    }
    return TN_SUCCESS;
}

/* ------------------------------------------------------------------ data movement ------ */

/* src/cpu/reps.cpp:16-97: the result is dense; for every index of the dimensions before `axis`,
 * every element j of the axis is written `reps` times in a row, each time with the whole inner
 * block that follows the axis. Source offsets honour the source's strides. */
tn_status orc_repeat(const tn_tensor_t* s, tn_tensor_t* d, int axis, int reps) {
    const size_t esize = dtype_bytes((int)s->dtype);
    if (s->dtype != d->dtype || esize == 0) return TN_UNSUPPORTED_DTYPE;
    const int rank = s->rank;
    if (axis < 0 || axis >= rank || reps < 1) return TN_ERROR;
    size_t outer = 1, inner = 1;
    for (int i = 0; i < axis; ++i) outer *= s->shape.sizes[i];
    for (int i = axis + 1; i < rank; ++i) inner *= s->shape.sizes[i];
    char* out = (char*)d->address;
    for (size_t o = 0; o < outer; ++o) {
        int64_t obase = 0;
        size_t t = o;
        for (int i = axis - 1; i >= 0; --i) {
            obase += (int64_t)(t % s->shape.sizes[i]) * s->strides.sizes[i];
            t /= s->shape.sizes[i];
        }
        for (size_t j = 0; j < s->shape.sizes[axis]; ++j) {
            for (int r = 0; r < reps; ++r) {
                for (size_t k = 0; k < inner; ++k) {
                    int64_t off = obase + (int64_t)j * s->strides.sizes[axis];
                    size_t tk = k;
                    for (int i = rank - 1; i > axis; --i) {
                        off += (int64_t)(tk % s->shape.sizes[i]) * s->strides.sizes[i];
                        tk /= s->shape.sizes[i];
                    }
                    memcpy(out, (const char*)s->address + off * (int64_t)esize, esize);
                    out += esize;
                }
            }
        }
    }
    return TN_SUCCESS;
}

/* src/cpu/concat.cpp:15-127: dense result; per index of the dimensions before `axis`, the block
 * of a, then the block of b. The inner block is walked through the operand's own strides for
 * every trailing dimension (the reference multiplies a flat inner index by the stride of
 * dimension axis + 1 alone, which is the same thing only for axis >= rank - 2). */
tn_status orc_concat(const tn_tensor_t* a, const tn_tensor_t* b, tn_tensor_t* d, int axis) {
    const size_t esize = dtype_bytes((int)d->dtype);
    if (a->dtype != d->dtype || b->dtype != d->dtype || esize == 0) return TN_UNSUPPORTED_DTYPE;
    const int rank = d->rank;
    if (axis < 0 || axis >= rank) return TN_ERROR;
    size_t outer = 1, inner = 1;
    for (int i = 0; i < axis; ++i) outer *= d->shape.sizes[i];
    for (int i = axis + 1; i < rank; ++i) inner *= d->shape.sizes[i];
    char* out = (char*)d->address;
    for (size_t o = 0; o < outer; ++o) {
        for (int which = 0; which < 2; ++which) {
            const tn_tensor_t* s = which ? b : a;
            int64_t obase = 0;
            size_t t = o;
            for (int i = axis - 1; i >= 0; --i) {
                obase += (int64_t)(t % s->shape.sizes[i]) * s->strides.sizes[i];
                t /= s->shape.sizes[i];
            }
            for (size_t j = 0; j < s->shape.sizes[axis]; ++j) {
                for (size_t k = 0; k < inner; ++k) {
                    int64_t off = obase + (int64_t)j * s->strides.sizes[axis];
                    size_t tk = k;
                    for (int i = rank - 1; i > axis; --i) {
                        off += (int64_t)(tk % s->shape.sizes[i]) * s->strides.sizes[i];
                        tk /= s->shape.sizes[i];
                    }
                    memcpy(out, (const char*)s->address + off * (int64_t)esize, esize);
                    out += esize;
                }
            }
        }
    }
    return TN_SUCCESS;
}

/* src/cpu/triang.cpp:3-103: matrices; upper keeps j >= i + k, lower keeps j <= i + k, every other
 * element becomes zero. i + k in signed arithmetic (the reference's unsigned sum differs for k < 0). */
tn_status orc_triangular(const tn_tensor_t* s, tn_tensor_t* d, int upper, int k) {
    const size_t esize = dtype_bytes((int)s->dtype);
    if (s->rank != 2 || d->rank != 2 || s->dtype != d->dtype || !is_numeric((int)s->dtype)) return TN_UNSUPPORTED_DTYPE;
    for (int64_t i = 0; i < (int64_t)s->shape.sizes[0]; ++i) {
        for (int64_t j = 0; j < (int64_t)s->shape.sizes[1]; ++j) {
            const int keep = upper ? (j >= i + k) : (j <= i + k);
            char* out = (char*)d->address + (i * d->strides.sizes[0] + j * d->strides.sizes[1]) * (int64_t)esize;
            if (keep) memcpy(out, (const char*)s->address + (i * s->strides.sizes[0] + j * s->strides.sizes[1]) * (int64_t)esize, esize);
            else memset(out, 0, esize);
        }
    }
    return TN_SUCCESS;
}

/* src/cpu/complex.cpp:14-228: complex result (interleaved, dense) from two real tensors of the same
 * rank with size-1 broadcasting; polar = (rho cos theta, rho sin theta). float32 arithmetic unless a
 * part is float64. */
tn_status orc_complex_pair(const tn_tensor_t* a, const tn_tensor_t* b, tn_tensor_t* d, int polar) {
    const int wide = a->dtype == TN_FLOAT64 || b->dtype == TN_FLOAT64;
    if ((int)d->dtype != (wide ? TN_COMPLEX128 : TN_COMPLEX64)) return TN_UNSUPPORTED_DTYPE;
    const int rank = d->rank;
    size_t cnt[TN_MAX_RANK] = {0};
    for (size_t idx = 0; idx < d->size; ++idx) {
        int64_t oa = 0, ob = 0;
        for (int dim = 0; dim < rank; ++dim) {
            oa += (int64_t)(a->shape.sizes[dim] == 1 ? 0 : cnt[dim]) * a->strides.sizes[dim];
            ob += (int64_t)(b->shape.sizes[dim] == 1 ? 0 : cnt[dim]) * b->strides.sizes[dim];
        }
        if (wide) {
            const double x = load_f64(a->address, (int)a->dtype, oa), y = load_f64(b->address, (int)b->dtype, ob);
            double* out = (double*)d->address + 2 * idx;
            out[0] = polar ? x * cos(y) : x;
            out[1] = polar ? x * sin(y) : y;
        } else {
            const float x = load_f32(a->address, (int)a->dtype, oa), y = load_f32(b->address, (int)b->dtype, ob);
            float* out = (float*)d->address + 2 * idx;
            out[0] = polar ? x * cosf(y) : x;
            out[1] = polar ? x * sinf(y) : y;
        }
        for (int dim = rank - 1; dim >= 0; --dim) {
            if (++cnt[dim] < d->shape.sizes[dim]) break;
            cnt[dim] = 0;
        }
    }
    return TN_SUCCESS;
}

/* ------------------------------------------------------------------ input generator ---- */

/* Counter-based generator shared by the tests and the benchmark so that host and device runs
 * see identical bits: splitmix64 of (seed, index) -> uniform in [0, 1). Not part of the
 * reference (it has no generator); documented here because the oracle's inputs come from it. */
static uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}
static double unit(uint64_t seed, uint64_t i) { return (double)(splitmix64(seed * 0xD1342543DE82EF95ull + i) >> 11) * (1.0 / 9007199254740992.0); }

/* kind 0: uniform [lo, hi); kind 1: normal(mean = lo, std = hi) by Box-Muller; integers:
 * uniform integers in [lo, hi]. Writes `n` elements of dtype `dt`, half types rounded RNE.
 * Element k of the output carries the value of counter `first + k`, so a slice of a larger
 * tensor can be generated on its own (a rank's shard; a chunk per host thread). */
tn_status orc_fill_range(void* dst, int dt, uint64_t first, size_t n, uint64_t seed, int kind, double lo, double hi) {
    if (!is_numeric(dt)) return TN_UNSUPPORTED_DTYPE;
    for (size_t k = 0; k < n; ++k) {
        const uint64_t i = first + k;
        double v;
        if (is_int(dt)) {
            const double span = hi - lo + 1.0;
            v = lo + floor(unit(seed, i) * span);
            store_i64(dst, dt, (int64_t)k, (int64_t)v);
            continue;
        }
        if (kind == 0) v = lo + (hi - lo) * unit(seed, i);
        else {
            double u1 = unit(seed, 2 * i), u2 = unit(seed, 2 * i + 1);
            if (u1 < 1e-300) u1 = 1e-300;
            v = lo + hi * sqrt(-2.0 * log(u1)) * cos(6.283185307179586 * u2);
        }
        if (dt == TN_FLOAT64) ((double*)dst)[k] = v;
        else store_f32(dst, dt, (int64_t)k, (float)v);
    }
    return TN_SUCCESS;
}

tn_status orc_fill(void* dst, int dt, size_t n, uint64_t seed, int kind, double lo, double hi) {
    return orc_fill_range(dst, dt, 0, n, seed, kind, lo, hi);
}
