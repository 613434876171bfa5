// tn_gemm / tn_gemm_scaled: shape and stride analysis, choice between the tcgen05 kernel
// (16-bit operands that TMA can address) and the SIMT kernel (everything else: fp32/fp64,
// integers, mixed pairs, odd pitches). Replaces src/cuda/matmul.cu of the reference.
#include "gemm_tc.cuh"

namespace tnb {

bool read_host_scalar(const tn_scalar_t* sc, double* f, int64_t* i);
tn_status tc_abort_count(unsigned int* count);
void tc_path_launches(uint64_t (&out)[4]);
tn_status reduce_abort_count(unsigned int* count);
tn_status tc_wait_probe(cudaStream_t stream, unsigned int polls);

tn_status surface_device_aborts() {
    static std::atomic<unsigned int> seen[64];
    int dev = 0;
    TN_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return TN_SUCCESS;
    unsigned int tc = 0, red = 0;
    TN_TRY(tc_abort_count(&tc));
    TN_TRY(reduce_abort_count(&red));
    const unsigned int total = tc + red, before = seen[dev].exchange(total);
    if (total > before)
        return fail(TN_ERROR, "%u thread block(s) on device %d gave up on a bounded device-side wait since the last synchronising call; "
                              "results written by those launches are incomplete", total - before, dev);
    return TN_SUCCESS;
}

namespace {

constexpr int kMaxBatchDims = TN_MAX_RANK - 2;

struct SimtArgs {
    const void* a;
    const void* b;
    void* d;
    int adt, bdt, ddt;
    int64_t M, N, K;
    int64_t a_sm, a_sk, b_sk, b_sn, d_sm, d_sn;  // element strides of the matrix dims
    int nbatch;                                  // number of batch dims
    int64_t batches;
    int64_t bsize[kMaxBatchDims];
    int64_t a_bs[kMaxBatchDims], b_bs[kMaxBatchDims], d_bs[kMaxBatchDims];
    int has_scale;
    double scale_f;
    int64_t scale_i;
    const int* run_if;  // when set: the kernel does nothing unless *run_if != 0 (device-side fallback)
};

constexpr int TM = 64, TN = 64, TK = 16;

// 64x64 tile per CTA of 256 threads, 4x4 outputs per thread, operands converted to the
// accumulator type C while they are staged in shared memory. Accumulation over k is in
// ascending order inside each thread, as in the reference loop (src/cpu/matmul.cpp:21-41).
template <typename C>
__global__ void __launch_bounds__(256) gemm_simt(const __grid_constant__ SimtArgs g) {
    __shared__ C As[TK][TM + 1];
    __shared__ C Bs[TK][TN + 1];
    if (g.run_if != nullptr && *g.run_if == 0) return;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    for (int64_t batch = blockIdx.z; batch < g.batches; batch += gridDim.z) {
        int64_t oa = 0, ob = 0, od = 0, rem = batch;
        for (int dim = g.nbatch - 1; dim >= 0; --dim) {
            const int64_t c = rem % g.bsize[dim];
            rem /= g.bsize[dim];
            oa += c * g.a_bs[dim];
            ob += c * g.b_bs[dim];
            od += c * g.d_bs[dim];
        }
        const int64_t m0 = (int64_t)blockIdx.y * TM, n0 = (int64_t)blockIdx.x * TN;
        C acc[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = C(0);
        for (int64_t k0 = 0; k0 < g.K; k0 += TK) {
            // 64x16 elements of A and 16x64 of B: 4 of each per thread
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int idx = threadIdx.x + e * 256;
                {
                    const int kk = idx & 15, mm = idx >> 4;  // k fastest: suits K-contiguous A
                    const int64_t m = m0 + mm, k = k0 + kk;
                    As[kk][mm] = (m < g.M && k < g.K) ? load_as<C>(g.a, g.adt, oa + m * g.a_sm + k * g.a_sk) : C(0);
                }
                {
                    int kk, nn;
                    if (g.b_sn == 1) { nn = idx & 63; kk = idx >> 6; }  // n fastest: N-contiguous B
                    else { kk = idx & 15; nn = idx >> 4; }               // k fastest: K-contiguous B
                    const int64_t n = n0 + nn, k = k0 + kk;
                    Bs[kk][nn] = (n < g.N && k < g.K) ? load_as<C>(g.b, g.bdt, ob + k * g.b_sk + n * g.b_sn) : C(0);
                }
            }
            __syncthreads();
#pragma unroll
            for (int kk = 0; kk < TK; ++kk) {
                C av[4], bv[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
#pragma unroll
                for (int j = 0; j < 4; ++j) bv[j] = Bs[kk][tx * 4 + j];
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if constexpr (std::is_same<C, int64_t>::value)
                            acc[i][j] = (int64_t)((uint64_t)acc[i][j] + (uint64_t)av[i] * (uint64_t)bv[j]);
                        else
                            acc[i][j] += av[i] * bv[j];
                    }
            }
            __syncthreads();
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int64_t m = m0 + ty * 4 + i;
            if (m >= g.M) continue;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int64_t n = n0 + tx * 4 + j;
                if (n >= g.N) continue;
                const int64_t off = od + m * g.d_sm + n * g.d_sn;
                if (g.has_scale) {
                    // round to the result dtype, multiply by the scalar, round again
                    store_as<C>(g.d, g.ddt, off, acc[i][j]);
                    C r = load_as<C>(g.d, g.ddt, off);
                    if constexpr (std::is_same<C, int64_t>::value) r = (int64_t)((uint64_t)r * (uint64_t)g.scale_i);
                    else r = r * static_cast<C>(g.scale_f);
                    store_as<C>(g.d, g.ddt, off, r);
                } else {
                    store_as<C>(g.d, g.ddt, off, acc[i][j]);
                }
            }
        }
    }
}

// Operand pairs of the reference's table (src/cpu/matmul.cpp:189-252).
bool pair_supported(int a, int b) {
    if (!is_numeric(a) || !is_numeric(b)) return false;
    if (is_int(a) && is_int(b)) return true;
    auto half_ok = [](int h, int o) { return o == h || o == TN_FLOAT32 || o == TN_FLOAT64 || is_int(o); };
    if (is_half(a)) return half_ok(a, b);
    if (is_half(b)) return half_ok(b, a);
    auto wide_ok = [](int o) { return o == TN_FLOAT32 || o == TN_FLOAT64 || o == TN_INT32; };
    return wide_ok(a) && wide_ok(b);
}

int compute_class(int a, int b) {
    if (a == TN_FLOAT64 || b == TN_FLOAT64) return 2;
    const bool fa = is_float(a), fb = is_float(b);
    if ((fa && b == TN_INT64) || (fb && a == TN_INT64)) return 2;
    if (fa || fb) return 1;
    return 0;
}

// ---- float32 operands on the tensor cores: three-way bfloat16 split -------------------------
// x = x0 + x1 + x2 with every part a bfloat16 (x0 = bf16(x), x1 = bf16(x - x0), x2 = bf16(x - x0 - x1);
// bfloat16 has float32's exponent range, so the parts carry 24 significand bits between them).
// A.B is then the sum of the six products A_i.B_j with i + j <= 2 (the others are below 2^-24 of
// the result), evaluated as ONE bfloat16 GEMM with float32 accumulation whose K extent is six times
// as long: A' = [A0 A0 A1 A0 A1 A2] and B' = [B0 B1 B0 B2 B1 B0] along K.
constexpr int kSplitTerms = 6;
__constant__ int kSplitA[kSplitTerms] = {0, 0, 1, 0, 1, 2};
__constant__ int kSplitB[kSplitTerms] = {0, 1, 0, 2, 1, 0};

__device__ __forceinline__ void split3(float x, uint16_t (&part)[3], int* non_finite) {
    if (!isfinite(x)) *non_finite = 1;  // benign race: every writer stores the same value
    __nv_bfloat16 p0 = __float2bfloat16_rn(x);
    if (isinf(__bfloat162float(p0)) && !isinf(x)) p0 = __ushort_as_bfloat16(x < 0 ? 0xFF7Fu : 0x7F7Fu);  // rounding overflowed
    float r = x - __bfloat162float(p0);
    if (!isfinite(x)) r = 0.0f;  // inf / NaN live in the first part alone
    const __nv_bfloat16 p1 = __float2bfloat16_rn(r);
    r -= __bfloat162float(p1);
    const __nv_bfloat16 p2 = __float2bfloat16_rn(r);
    part[0] = __bfloat16_as_ushort(p0);
    part[1] = __bfloat16_as_ushort(p1);
    part[2] = __bfloat16_as_ushort(p2);
}

// x[batch][r][k] (any strides) -> out[batch][r][6 * kp], k fastest on the way out; columns k >= K are zero.
__global__ void __launch_bounds__(256) split_k_major(const float* __restrict__ x, uint16_t* __restrict__ out, int64_t rows, int64_t K,
                                                     int64_t kp, int64_t s_r, int64_t s_k, int64_t s_batch, int second_operand, int* non_finite) {
    const int64_t batch = blockIdx.z;
    const float* xb = x + batch * s_batch;
    uint16_t* ob = out + batch * rows * kSplitTerms * kp;
    const int64_t n = rows * kp;
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (int64_t)gridDim.x * 256) {
        const int64_t r = i / kp, k = i - r * kp;
        uint16_t part[3] = {0, 0, 0};
        if (k < K) split3(xb[r * s_r + k * s_k], part, non_finite);
#pragma unroll
        for (int t = 0; t < kSplitTerms; ++t) ob[r * kSplitTerms * kp + t * kp + k] = part[second_operand ? kSplitB[t] : kSplitA[t]];
    }
}

// b[batch][k][n] with n contiguous -> out[batch][6 * kp][np], n fastest; rows k >= K and columns n >= N are zero.
__global__ void __launch_bounds__(256) split_n_major(const float* __restrict__ b, uint16_t* __restrict__ out, int64_t K, int64_t N,
                                                     int64_t kp, int64_t np, int64_t s_k, int64_t s_batch, int* non_finite) {
    const int64_t batch = blockIdx.z;
    const float* bb = b + batch * s_batch;
    uint16_t* ob = out + batch * kSplitTerms * kp * np;
    const int64_t n_all = kp * np;
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n_all; i += (int64_t)gridDim.x * 256) {
        const int64_t k = i / np, n = i - k * np;
        uint16_t part[3] = {0, 0, 0};
        if (k < K && n < N) split3(bb[k * s_k + n], part, non_finite);
#pragma unroll
        for (int t = 0; t < kSplitTerms; ++t) ob[(t * kp + k) * np + n] = part[kSplitB[t]];
    }
}

// Row statistics of the result requested together with the product (tn_gemm_scaled_stats).
struct StatsRequest {
    tn_tensor_t* max = nullptr;
    tn_tensor_t* sum = nullptr;
    tn_tensor_t* argmax = nullptr;
    bool any() const { return max || sum || argmax; }
    // tn_gemm_mirrored: further result buffers (peer memory) the epilogue writes as well; `mirrored` reports
    // whether the kernel that can do that took the product
    void* mirrors[7] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    int n_mirrors = 0;
    bool* mirrored = nullptr;
};

tn_status gemm_impl(const tn_tensor_t* a, const tn_tensor_t* b, tn_tensor_t* dst, const tn_scalar_t* scale,
                    tn_stream_t stream, const StatsRequest* stats = nullptr, bool* stats_done = nullptr) {
    if (!a || !b || !dst) return fail(TN_ERROR, "null tensor");
    if (!pair_supported(a->dtype, b->dtype) || !is_numeric(dst->dtype))
        return fail(TN_UNSUPPORTED_DTYPE, "gemm: dtype pair (%d, %d) -> %d unsupported", (int)a->dtype, (int)b->dtype,
                    (int)dst->dtype);
    if (a->rank < 2 || b->rank < 2 || dst->rank < 2)
        return fail(TN_ERROR, "gemm: operands must have rank >= 2 (got %d, %d -> %d)", (int)a->rank, (int)b->rank, (int)dst->rank);
    if (a->environment.kind != TN_DEVICE || b->environment.kind != TN_DEVICE ||
        a->environment.resource.device.id != b->environment.resource.device.id ||
        a->environment.resource.device.id != dst->environment.resource.device.id)
        return fail(TN_INCOMPATIBLE_DEVICES, "operands must live on one device");
    TN_TRY(use_device_of(dst));

    SimtArgs g;
    g.a = a->address;
    g.b = b->address;
    g.d = dst->address;
    g.adt = a->dtype;
    g.bdt = b->dtype;
    g.ddt = dst->dtype;
    const int ra = a->rank, rb = b->rank, rd = dst->rank;
    g.M = (int64_t)dst->shape.sizes[rd - 2];
    g.N = (int64_t)dst->shape.sizes[rd - 1];
    g.K = (int64_t)a->shape.sizes[ra - 1];
    if ((int64_t)a->shape.sizes[ra - 2] != g.M || (int64_t)b->shape.sizes[rb - 1] != g.N ||
        (int64_t)b->shape.sizes[rb - 2] != g.K)
        return fail(TN_ERROR, "gemm: shapes do not contract ([%lld,%lld] x [%lld,%lld] -> [%lld,%lld])",
                    (long long)a->shape.sizes[ra - 2], (long long)g.K, (long long)b->shape.sizes[rb - 2],
                    (long long)b->shape.sizes[rb - 1], (long long)g.M, (long long)g.N);
    g.a_sm = a->strides.sizes[ra - 2];
    g.a_sk = a->strides.sizes[ra - 1];
    g.b_sk = b->strides.sizes[rb - 2];
    g.b_sn = b->strides.sizes[rb - 1];
    g.d_sm = dst->strides.sizes[rd - 2];
    g.d_sn = dst->strides.sizes[rd - 1];
    g.nbatch = rd - 2;
    g.batches = 1;
    for (int dim = 0; dim < g.nbatch; ++dim) {
        g.bsize[dim] = (int64_t)dst->shape.sizes[dim];
        g.batches *= g.bsize[dim];
        g.d_bs[dim] = dst->strides.sizes[dim];
        // batch dims broadcast NumPy-style: missing or extent-1 dims reuse the operand
        // (src/cpu/matmul.cpp:96-124)
        const int da = dim + (ra - rd), db = dim + (rb - rd);
        g.a_bs[dim] = (da >= 0 && da < ra - 2 && a->shape.sizes[da] != 1) ? a->strides.sizes[da] : 0;
        g.b_bs[dim] = (db >= 0 && db < rb - 2 && b->shape.sizes[db] != 1) ? b->strides.sizes[db] : 0;
        if (da >= 0 && da < ra - 2 && a->shape.sizes[da] != 1 && (int64_t)a->shape.sizes[da] != g.bsize[dim])
            return fail(TN_ERROR, "gemm: batch dim %d of the first operand does not broadcast", dim);
        if (db >= 0 && db < rb - 2 && b->shape.sizes[db] != 1 && (int64_t)b->shape.sizes[db] != g.bsize[dim])
            return fail(TN_ERROR, "gemm: batch dim %d of the second operand does not broadcast", dim);
    }
    g.has_scale = 0;
    g.scale_f = 1.0;
    g.scale_i = 1;
    g.run_if = nullptr;
    if (scale) {
        if (scale->dtype != dst->dtype) return fail(TN_UNSUPPORTED_DTYPE, "gemm_scaled: scalar dtype %d, result dtype %d", (int)scale->dtype, (int)dst->dtype);
        if (!read_host_scalar(scale, &g.scale_f, &g.scale_i)) return fail(TN_ERROR, "gemm_scaled: unreadable scalar");
        g.has_scale = 1;
    }
    if (g.M == 0 || g.N == 0 || g.batches == 0) return TN_SUCCESS;
    cudaStream_t s = as_cuda(stream);

    // collapse the batch dims of an operand into one stride; possible when walking them in row-major
    // order advances by a constant stride, or the operand is shared by every batch
    auto collapse_in = [](const SimtArgs& q, const int64_t* bs, int64_t* stride) {
        bool any = false, all = true;
        int64_t expect = 0;
        for (int dim = q.nbatch - 1; dim >= 0; --dim) {
            if (q.bsize[dim] == 1) continue;
            if (bs[dim] == 0) { all = false; continue; }
            if (!any) { expect = bs[dim]; *stride = bs[dim]; any = true; }
            if (bs[dim] != expect) return false;
            expect = bs[dim] * q.bsize[dim];
        }
        if (!any) { *stride = 0; return true; }
        return all;
    };
    auto collapse_batches = [&](const int64_t* bs, int64_t* stride) { return collapse_in(g, bs, stride); };

    // ---- float32 on the tensor cores (three-way bfloat16 split), for products big enough to pay for
    //      the split passes: dense rows in the result, batch dims that collapse
    static const bool f32_on_tc = !getenv("TN_GEMM_F32_SIMT");
    if (f32_on_tc && a->dtype == TN_FLOAT32 && b->dtype == TN_FLOAT32 && dst->dtype == TN_FLOAT32 && g.d_sn == 1 && g.K > 0 &&
        (double)g.batches * (double)g.M * (double)g.N * (double)g.K >= (double)(1 << 24) && g.batches <= 65535) {
        int64_t sa = 0, sb = 0, sd = 0;
        if (collapse_batches(g.a_bs, &sa) && collapse_batches(g.b_bs, &sb) && collapse_batches(g.d_bs, &sd) && (sd != 0 || g.batches == 1)) {
            const int64_t kp = (g.K + 7) & ~int64_t(7), np = (g.N + 7) & ~int64_t(7);
            const bool b_n_major = g.b_sn == 1 && g.b_sk != 1;
            const int64_t a_copies = sa ? g.batches : 1, b_copies = sb ? g.batches : 1;
            const size_t a_elems = (size_t)a_copies * g.M * kSplitTerms * kp;
            const size_t b_elems = (size_t)b_copies * kSplitTerms * kp * (b_n_major ? np : g.N);
            const size_t a_bytes = (a_elems * 2 + 255) & ~size_t(255), b_bytes = b_elems * 2;
            if (a_bytes + b_bytes <= (size_t(8) << 30) && ceil_div(g.M, TM) <= 65535) {
                uint8_t* scratch = nullptr;
                TN_TRY(scratch_alloc(reinterpret_cast<void**>(&scratch), a_bytes + b_bytes + 256, s));
                uint16_t* a3 = reinterpret_cast<uint16_t*>(scratch);
                uint16_t* b3 = reinterpret_cast<uint16_t*>(scratch + a_bytes);
                // An infinity or NaN cannot go through the split (inf times the parts of the other operand
                // gives infinities of both signs). The split passes raise this flag when they meet one, and
                // the element-wise kernel, launched behind the tensor-core GEMM, recomputes the product only
                // if the flag is up: no host round trip, one near-empty launch otherwise.
                int* non_finite = reinterpret_cast<int*>(scratch + a_bytes + ((b_bytes + 255) & ~size_t(255)));
                if (cudaMemsetAsync(non_finite, 0, sizeof(int), s) != cudaSuccess) {
                    scratch_free(scratch, s);
                    return fail(TN_ERROR, "gemm: could not clear the fallback flag");
                }
                const int blocks = sm_count() * 8;
                split_k_major<<<dim3((unsigned)std::min<int64_t>(blocks, ceil_div(g.M * kp, 256)), 1, (unsigned)a_copies), 256, 0, s>>>(
                    static_cast<const float*>(g.a), a3, g.M, g.K, kp, g.a_sm, g.a_sk, sa, 0, non_finite);
                tn_status st = after_launch("split_k_major");
                if (st == TN_SUCCESS) {
                    if (b_n_major)
                        split_n_major<<<dim3((unsigned)std::min<int64_t>(blocks, ceil_div(kp * np, 256)), 1, (unsigned)b_copies), 256, 0, s>>>(
                            static_cast<const float*>(g.b), b3, g.K, g.N, kp, np, g.b_sk, sb, non_finite);
                    else
                        split_k_major<<<dim3((unsigned)std::min<int64_t>(blocks, ceil_div(g.N * kp, 256)), 1, (unsigned)b_copies), 256, 0, s>>>(
                            static_cast<const float*>(g.b), b3, g.N, g.K, kp, g.b_sn, g.b_sk, sb, 1, non_finite);
                    st = after_launch("split operand");
                }
                if (st == TN_SUCCESS) {
                    TcGemm p;
                    p.a = a3;
                    p.b = b3;
                    p.d = g.d;
                    p.ab_dtype = TN_BFLOAT16;
                    p.d_dtype = TN_FLOAT32;
                    p.M = g.M;
                    p.N = g.N;
                    p.K = kSplitTerms * kp;
                    p.lda = kSplitTerms * kp;
                    p.b_n_major = b_n_major;
                    p.ldb = b_n_major ? np : kSplitTerms * kp;
                    p.ldd = g.d_sm;
                    p.batches = g.batches;
                    p.a_batch = sa ? g.M * kSplitTerms * kp : 0;
                    p.b_batch = sb ? kSplitTerms * kp * (b_n_major ? np : g.N) : 0;
                    p.d_batch = sd;
                    p.has_scale = g.has_scale != 0;
                    p.scale = (float)g.scale_f;
                    st = tc_gemm_eligible(p) ? tc_gemm(p, s) : TN_UNSUPPORTED_DTYPE;
                    const int64_t gy = ceil_div(g.M, TM);
                    if (st == TN_SUCCESS && gy <= 65535) {
                        SimtArgs guarded = g;
                        guarded.run_if = non_finite;
                        const dim3 grid((unsigned)ceil_div(g.N, TN), (unsigned)gy, (unsigned)g.batches);
                        gemm_simt<float><<<grid, 256, 0, s>>>(guarded);
                        st = after_launch("gemm_simt (non-finite fallback)");
                    }
                }
                const tn_status fr = scratch_free(scratch, s);
                if (st == TN_SUCCESS) return fr;
                if (st != TN_UNSUPPORTED_DTYPE) return st;  // else: not addressable by TMA, take the SIMT kernel
            }
        }
    }

    // ---- tensor-core path: 16-bit operands of one type, result of that type or fp32,
    //      row-major result, batch dims that collapse to one stride per operand.
    // Returns TN_SUCCESS with *launched = false when the problem `q` is not one the kernel addresses.
    auto half_on_tensor_cores = [&](const SimtArgs& q, bool with_stats, bool* launched) -> tn_status {
        *launched = false;
        int64_t sa = 0, sb = 0, sd = 0;
        if (!(collapse_in(q, q.a_bs, &sa) && collapse_in(q, q.b_bs, &sb) && collapse_in(q, q.d_bs, &sd) && (sd != 0 || q.batches == 1)))
            return TN_SUCCESS;
        TcGemm p;
        p.a = q.a;
        p.b = q.b;
        p.d = q.d;
        p.ab_dtype = a->dtype;
        p.d_dtype = dst->dtype;
        p.M = q.M;
        p.N = q.N;
        p.K = q.K;
        p.lda = q.a_sm;
        p.b_n_major = q.b_sk != 1;  // then b_sn == 1: rows of B are N-contiguous
        p.ldb = p.b_n_major ? q.b_sk : q.b_sn;
        p.ldd = q.d_sm;
        p.batches = q.batches;
        p.a_batch = sa;
        p.b_batch = sb;
        p.d_batch = sd;
        // [B, M, K] x shared [K, N] with dense A and D folds into one tall GEMM
        if (q.batches > 1 && sb == 0 && sa == q.M * q.a_sm && sd == q.M * q.d_sm) {
            p.M = q.M * q.batches;
            p.batches = 1;
            p.a_batch = p.d_batch = 0;
        }
        p.has_scale = q.has_scale != 0;
        p.scale = (float)q.scale_f;
        if (with_stats && stats && stats->any() && tc_gemm_can_fuse_stats(p)) {
            // the epilogue keeps each row's maximum, sum and argmax while it drains the row
            p.stat_max = stats->max ? stats->max->address : nullptr;
            p.stat_sum = stats->sum ? stats->sum->address : nullptr;
            p.stat_argmax = stats->argmax ? static_cast<int64_t*>(stats->argmax->address) : nullptr;
            if (stats_done) *stats_done = true;
        }
        if (with_stats && stats && stats->n_mirrors > 0) {
            for (int m = 0; m < stats->n_mirrors; ++m) p.mirrors[m] = stats->mirrors[m];
            p.n_mirrors = stats->n_mirrors;
        }
        if (tc_gemm_eligible(p)) {
            *launched = true;
            TN_TRY(tc_gemm(p, s));
            if (p.n_mirrors > 0 && stats->mirrored) *stats->mirrored = true;
            return TN_SUCCESS;
        }
        if (with_stats && stats_done) *stats_done = false;
        return TN_SUCCESS;
    };
    if (a->dtype == b->dtype && is_half(a->dtype) && (dst->dtype == a->dtype || dst->dtype == TN_FLOAT32) &&
        g.a_sk == 1 && g.d_sn == 1 && (g.b_sk == 1 || g.b_sn == 1) && g.K > 0) {
        bool launched = false;
        TN_TRY(half_on_tensor_cores(g, true, &launched));
        if (launched) return TN_SUCCESS;
        // Batch dims that do not collapse as a whole (an operand that broadcasts over SOME of them:
        // [2,1,M,K] x [2,3,K,N]) usually do once the outermost one is peeled off: one launch per
        // index of that dim, each a batched problem over the remaining dims.
        int outer = 0;
        while (outer < g.nbatch && g.bsize[outer] == 1) ++outer;
        if (outer < g.nbatch && g.bsize[outer] <= 64 && g.batches > g.bsize[outer]) {
            const int64_t es = 2, ds = dst->dtype == TN_FLOAT32 ? 4 : 2;
            auto slice = [&](int64_t i) {
                SimtArgs q = g;
                q.a = static_cast<const uint8_t*>(g.a) + i * g.a_bs[outer] * es;
                q.b = static_cast<const uint8_t*>(g.b) + i * g.b_bs[outer] * es;
                q.d = static_cast<uint8_t*>(g.d) + i * g.d_bs[outer] * ds;
                q.batches = g.batches / g.bsize[outer];
                q.bsize[outer] = 1;
                return q;
            };
            // every slice has the same shape and strides; they differ in their base addresses only, and
            // those stay 16-byte aligned when the peeled strides are multiples of 8 elements
            const bool aligned = g.a_bs[outer] % 8 == 0 && g.b_bs[outer] % 8 == 0 && g.d_bs[outer] % 8 == 0;
            if (aligned) {
                TN_TRY(half_on_tensor_cores(slice(0), false, &launched));
                if (launched) {
                    for (int64_t i = 1; i < g.bsize[outer]; ++i) {
                        bool again = false;
                        TN_TRY(half_on_tensor_cores(slice(i), false, &again));
                        if (!again) return fail(TN_ERROR, "gemm: slice %lld of a peeled batch dim was refused by the tensor-core path", (long long)i);
                    }
                    return TN_SUCCESS;
                }
            }
        }
    }

    // ---- SIMT path
    const int64_t gx = ceil_div(g.N, TN), gy = ceil_div(g.M, TM);
    if (gy > 65535) return fail(TN_ERROR, "gemm: M = %lld is too large for the SIMT path", (long long)g.M);
    const dim3 grid((unsigned)gx, (unsigned)gy, (unsigned)(g.batches < 65535 ? g.batches : 65535));
    switch (compute_class(a->dtype, b->dtype)) {
        case 2: gemm_simt<double><<<grid, 256, 0, s>>>(g); break;
        case 1: gemm_simt<float><<<grid, 256, 0, s>>>(g); break;
        default: gemm_simt<int64_t><<<grid, 256, 0, s>>>(g); break;
    }
    return after_launch("gemm_simt");
}

}  // namespace
}  // namespace tnb

using namespace tnb;

extern "C" {

// 16-bit operands whose layout the tensor-core path cannot address (first operand not K-contiguous,
// second neither K- nor N-contiguous, pitches that are not multiples of 16 bytes) are first copied
// into dense scratch tensors (the strided copy transposes through shared-memory tiles), when the
// product is big enough for the tensor cores to pay for that pass.
static bool tc_addressable(const tn_tensor_t* t, bool second) {
    const int r = t->rank;
    if (r < 2) return true;
    const int64_t s_row = t->strides.sizes[r - 2], s_col = t->strides.sizes[r - 1];
    const bool rows_ok = s_col == 1 && s_row % 8 == 0;                 // last dimension contiguous
    const bool cols_ok = second && s_row == 1 && s_col % 8 == 0;       // second operand as [N, K] seen transposed
    if (!(rows_ok || cols_ok) || (reinterpret_cast<uintptr_t>(t->address) & 15) != 0) return false;
    for (int d = 0; d < r - 2; ++d)
        if (t->shape.sizes[d] != 1 && t->strides.sizes[d] % 8 != 0) return false;
    return true;
}

static tn_status gemm_entry(const tn_tensor_t* a, const tn_tensor_t* b, tn_tensor_t* dst, const tn_scalar_t* scale, tn_stream_t stream,
                            const StatsRequest* stats = nullptr, bool* stats_done = nullptr) {
    if (a && b && dst && a->dtype == b->dtype && is_half(a->dtype) && a->rank >= 2 && b->rank >= 2 && dst->rank >= 2 &&
        a->environment.kind == TN_DEVICE && b->environment.kind == TN_DEVICE && dst->environment.kind == TN_DEVICE) {
        const bool fix_a = !tc_addressable(a, false), fix_b = !tc_addressable(b, true);
        const double work = (double)dst->size * (double)a->shape.sizes[a->rank - 1];
        if ((fix_a || fix_b) && work >= (double)(1 << 24) && a->shape.sizes[a->rank - 1] % 8 == 0 &&
            (!fix_b || b->shape.sizes[b->rank - 1] % 8 == 0)) {
            TN_TRY(use_device_of(dst));
            cudaStream_t s = as_cuda(stream);
            auto dense_copy = [&](const tn_tensor_t* t, tn_tensor_t* out, void** mem) -> tn_status {
                *out = *t;
                int64_t run = 1;
                for (int d = t->rank - 1; d >= 0; --d) {
                    out->strides.sizes[d] = run;
                    run *= (int64_t)t->shape.sizes[d];
                }
                out->layout = TN_CONTIGUOUS;
                TN_TRY(scratch_alloc(mem, (size_t)run * 2, s));
                out->address = *mem;
                return tn_cpy(t, out, stream);
            };
            tn_tensor_t da, db;
            void *ma = nullptr, *mb = nullptr;
            tn_status st = TN_SUCCESS;
            if (fix_a) st = dense_copy(a, &da, &ma);
            if (st == TN_SUCCESS && fix_b) st = dense_copy(b, &db, &mb);
            if (st == TN_SUCCESS) st = gemm_impl(fix_a ? &da : a, fix_b ? &db : b, dst, scale, stream, stats, stats_done);
            if (ma) scratch_free(ma, s);
            if (mb) scratch_free(mb, s);
            return st;
        }
    }
    return gemm_impl(a, b, dst, scale, stream, stats, stats_done);
}

tn_status tn_gemm(const tn_tensor_t* a, const tn_tensor_t* b, tn_tensor_t* dst, tn_stream_t stream) {
    return gemm_entry(a, b, dst, nullptr, stream);
}

tn_status tn_gemm_scaled(const tn_tensor_t* a, const tn_tensor_t* b, const tn_scalar_t* scale, tn_tensor_t* dst,
                         tn_stream_t stream) {
    if (!scale) return fail(TN_ERROR, "null scalar");
    return gemm_entry(a, b, dst, scale, stream);
}

tn_status tn_gemm_scaled_stats(const tn_tensor_t* a, const tn_tensor_t* b, const tn_scalar_t* scale, tn_tensor_t* dst,
                               tn_tensor_t* max_out, tn_tensor_t* sum_out, tn_tensor_t* argmax_out, tn_stream_t stream) {
    if (!dst) return fail(TN_ERROR, "null tensor");
    if (!max_out && !sum_out && !argmax_out) return fail(TN_ERROR, "gemm_scaled_stats: no statistic requested");
    if (dst->rank < 2) return fail(TN_ERROR, "gemm_scaled_stats: the result must have rank >= 2");
    const size_t rows = dst->shape.sizes[dst->rank - 1] ? dst->size / dst->shape.sizes[dst->rank - 1] : 0;
    auto check_out = [&](const tn_tensor_t* t, int want_dtype, const char* what) -> tn_status {
        if (!t) return TN_SUCCESS;
        if ((int)t->dtype != want_dtype) return fail(TN_UNSUPPORTED_DTYPE, "gemm_scaled_stats: %s has dtype %d, expected %d", what, (int)t->dtype, want_dtype);
        if (t->size != rows) return fail(TN_ERROR, "gemm_scaled_stats: %s has %zu elements, the result has %zu rows", what, t->size, rows);
        if (t->environment.kind != TN_DEVICE || t->environment.resource.device.id != dst->environment.resource.device.id)
            return fail(TN_INCOMPATIBLE_DEVICES, "operands must live on one device");
        int64_t expect = 1;
        for (int d = t->rank - 1; d >= 0; --d) {
            if (t->shape.sizes[d] != 1 && t->strides.sizes[d] != expect) return fail(TN_ERROR, "gemm_scaled_stats: %s must be dense", what);
            expect *= (int64_t)t->shape.sizes[d];
        }
        return TN_SUCCESS;
    };
    TN_TRY(check_out(max_out, (int)dst->dtype, "max"));
    TN_TRY(check_out(sum_out, (int)dst->dtype, "sum"));
    TN_TRY(check_out(argmax_out, TN_INT64, "argmax"));
    StatsRequest request;
    request.max = max_out;
    request.sum = sum_out;
    request.argmax = argmax_out;
    bool fused = false;
    TN_TRY(gemm_entry(a, b, dst, scale, stream, &request, &fused));
    if (fused) return TN_SUCCESS;
    // shapes the fused epilogue does not cover: the statistics take their own pass over the result
    return tn_reduce_stats(dst, max_out, sum_out, argmax_out, stream, (uint8_t)(dst->rank - 1));
}

tn_status tn_device_errors(unsigned int* count) {
    if (!count) return fail(TN_ERROR, "null count");
    unsigned int tc = 0, red = 0;
    TN_TRY(tc_abort_count(&tc));
    TN_TRY(reduce_abort_count(&red));
    *count = tc + red;
    return TN_SUCCESS;
}

tn_status tn_gemm_mirrored(const tn_tensor_t* a, const tn_tensor_t* b, tn_tensor_t* dst, const tn_tensor_t* const* mirrors, int n_mirrors,
                           tn_stream_t stream) {
    if (!dst || (n_mirrors > 0 && !mirrors)) return fail(TN_ERROR, "null argument");
    if (n_mirrors < 0 || n_mirrors > 7) return fail(TN_ERROR, "gemm_mirrored: %d mirrors, at most 7", n_mirrors);
    StatsRequest request;
    bool mirrored = false;
    for (int m = 0; m < n_mirrors; ++m) {
        const tn_tensor_t* t = mirrors[m];
        if (!t) return fail(TN_ERROR, "gemm_mirrored: null mirror");
        bool same = t->rank == dst->rank && t->dtype == dst->dtype && t->environment.kind == TN_DEVICE;
        for (int d = 0; same && d < dst->rank; ++d) same = t->shape.sizes[d] == dst->shape.sizes[d] && t->strides.sizes[d] == dst->strides.sizes[d];
        if (!same) return fail(TN_ERROR, "gemm_mirrored: mirror %d must have the result's dtype, shape and strides", m);
        request.mirrors[m] = t->address;
    }
    request.n_mirrors = n_mirrors;
    request.mirrored = &mirrored;
    if (n_mirrors == 0) return gemm_entry(a, b, dst, nullptr, stream);
    bool unused = false;
    TN_TRY(gemm_entry(a, b, dst, nullptr, stream, &request, &unused));
    if (!mirrored)
        return fail(TN_ERROR, "gemm_mirrored: this product does not run on the tensor-core kernel that writes mirrors (16-bit operands and result, "
                              "16-byte aligned bases and pitches); the result was written to dst only");
    return TN_SUCCESS;
}

tn_status tn_gemm_path_launches(uint64_t counts[4]) {
    if (!counts) return fail(TN_ERROR, "null counts");
    uint64_t c[4];
    tc_path_launches(c);
    for (int i = 0; i < 4; ++i) counts[i] = c[i];
    return TN_SUCCESS;
}

tn_status tn_selftest_bounded_wait(const tn_device_t* device, tn_stream_t stream, unsigned int polls) {
    if (!device) return fail(TN_ERROR, "null device");
    TN_TRY(use_device(device->id));
    return tc_wait_probe(as_cuda(stream), polls);
}

}  // extern "C"
