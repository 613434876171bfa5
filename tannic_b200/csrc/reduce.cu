// Axis reductions: argmax / argmin (int64 index, first occurrence, NaN never selected),
// sum / mean (accumulate wider than storage), value max, and a fused max+sum+argmax pass.
// Replaces src/cuda/argred.cu of the reference (one thread per output, serial over the axis).
//
// Kernels:
//   reduce_rows_warp   dense source, last axis: one warp per row, 16-byte loads where the row
//                      is aligned, shuffle combine; rows may start at any element offset
//                      (197-wide bf16 rows have a 394-byte pitch);
//   reduce_rows_staged same geometry for SHORT rows (<= 1 KiB, e.g. the 197-wide score rows): a CTA
//                      brings a contiguous chunk of whole rows into shared memory with 16-byte
//                      asynchronous copies (double-buffered), then a few lanes reduce each row;
//   reduce_rows_block  same geometry for long rows: one CTA per row;
//   reduce_split       few, very long rows: every row is cut into segments whose partial
//                      results go to scratch memory, a second kernel combines them;
//   reduce_cols_tiled  dense source, inner axis: 32 x 8 thread tiles, 16-byte loads along the inner
//                      extent, the reduced axis split inside and across CTAs (partials in scratch);
//   reduce_cols        the same for a narrow inner extent: one thread per output column;
//   reduce_strided     any view: one thread per output.
#include "common.cuh"

#include <cfloat>
#include <climits>
#include <cstdlib>
#include <mutex>

namespace tnb {
namespace {

constexpr int kThreads = 256;
constexpr int64_t kNoIndex = INT64_MAX;

template <typename T> struct acc_of { using type = int64_t; };  // integers: int64 (src/cuda/argred.cu:167-187)
template <> struct acc_of<__half> { using type = float; };
template <> struct acc_of<__nv_bfloat16> { using type = float; };
template <> struct acc_of<float> { using type = double; };
template <> struct acc_of<double> { using type = double; };

template <typename T> struct cmp_of { using type = T; };
template <> struct cmp_of<__half> { using type = float; };
template <> struct cmp_of<__nv_bfloat16> { using type = float; };

template <typename C, bool MIN> __device__ __forceinline__ C cmp_init() {
    if constexpr (std::is_same<C, float>::value) return MIN ? INFINITY : -INFINITY;
    else if constexpr (std::is_same<C, double>::value) return MIN ? (double)INFINITY : -(double)INFINITY;
    else if constexpr (std::is_same<C, int8_t>::value) return MIN ? INT8_MAX : INT8_MIN;
    else if constexpr (std::is_same<C, int16_t>::value) return MIN ? INT16_MAX : INT16_MIN;
    else if constexpr (std::is_same<C, int32_t>::value) return MIN ? INT32_MAX : INT32_MIN;
    else return MIN ? INT64_MAX : INT64_MIN;
}

// 16-bit floats are read from shared memory two at a time as one 32-bit word.
template <typename T> struct is_half16 { static constexpr bool value = false; };
template <> struct is_half16<__half> { static constexpr bool value = true; };
template <> struct is_half16<__nv_bfloat16> { static constexpr bool value = true; };
template <typename T> struct pair_of_half { using type = __half2; };
template <> struct pair_of_half<__nv_bfloat16> { using type = __nv_bfloat162; };
// both halves of a word set to the 16-bit form of `v`
template <typename T> __device__ __forceinline__ uint32_t pair_bits(float v) {
    const T one = from_compute<T, float>(v);
    const uint32_t b = *reinterpret_cast<const uint16_t*>(&one);
    return b | (b << 16);
}
template <typename T> __device__ __forceinline__ float half_of_pair(uint32_t w, int h) {
    const uint16_t bits = static_cast<uint16_t>(h ? (w >> 16) : (w & 0xffffu));
    return to_compute<float>(*reinterpret_cast<const T*>(&bits));
}

// Running state of one lane. The lane visits its elements in ascending index order, so a
// strict comparison keeps the first occurrence; an element equal to the initial value never
// wins, which leaves index 0 for rows made of -inf / NaN only (src/cpu/argred.cpp:80-108).
template <typename T, bool SUM, bool ARG, bool MIN>
struct State {
    using A = typename acc_of<T>::type;
    using C = typename cmp_of<T>::type;
    A sum;
    C best;
    int64_t idx;
    __device__ __forceinline__ void init() {
        sum = A(0);
        best = cmp_init<C, MIN>();
        idx = kNoIndex;
    }
    __device__ __forceinline__ void feed(T raw, int64_t i) {
        if constexpr (SUM) sum += to_compute<A>(raw);
        if constexpr (ARG) {
            const C v = to_compute<C>(raw);
            if (MIN ? (v < best) : (v > best)) {
                best = v;
                idx = i;
            }
        }
    }
    __device__ __forceinline__ void merge(A osum, C obest, int64_t oidx) {
        if constexpr (SUM) sum += osum;
        if constexpr (ARG) {
            const bool better = MIN ? (obest < best) : (obest > best);
            if (better || (obest == best && oidx < idx)) {
                best = obest;
                idx = oidx;
            }
        }
    }
    __device__ __forceinline__ void merge(const State& o) { merge(o.sum, o.best, o.idx); }
};

template <typename V> __device__ __forceinline__ V shfl_xor(V v, int mask) { return __shfl_xor_sync(0xffffffffu, v, mask); }
template <> __device__ __forceinline__ int8_t shfl_xor<int8_t>(int8_t v, int mask) { return (int8_t)__shfl_xor_sync(0xffffffffu, (int)v, mask); }
template <> __device__ __forceinline__ int16_t shfl_xor<int16_t>(int16_t v, int mask) { return (int16_t)__shfl_xor_sync(0xffffffffu, (int)v, mask); }
template <> __device__ __forceinline__ int64_t shfl_xor<int64_t>(int64_t v, int mask) { return (int64_t)__shfl_xor_sync(0xffffffffu, (long long)v, mask); }

template <typename T, bool SUM, bool ARG, bool MIN>
__device__ __forceinline__ void warp_combine(State<T, SUM, ARG, MIN>& st) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) {
        typename State<T, SUM, ARG, MIN>::A osum = SUM ? shfl_xor(st.sum, m) : st.sum;
        typename State<T, SUM, ARG, MIN>::C obest = ARG ? shfl_xor(st.best, m) : st.best;
        int64_t oidx = ARG ? shfl_xor(st.idx, m) : st.idx;
        st.merge(osum, obest, oidx);
    }
}

struct Outputs {
    void* sum;      // storage dtype: sum or mean
    void* value;    // storage dtype: max / min value
    int64_t* index; // int64
    int mean;       // divide the sum by the axis length
};

template <typename T, bool SUM, bool ARG, bool MIN>
__device__ __forceinline__ void write_out(const State<T, SUM, ARG, MIN>& st, const Outputs& out, int64_t o, int64_t len,
                                          T first) {
    using A = typename acc_of<T>::type;
    if constexpr (SUM) {
        if (out.sum) {
            A s = st.sum;
            if (out.mean) s = s / static_cast<A>(len);
            static_cast<T*>(out.sum)[o] = from_compute<T, A>(s);
        }
    }
    if constexpr (ARG) {
        const bool none = st.idx == kNoIndex;
        if (out.index) out.index[o] = none ? 0 : st.idx;
        if (out.value) static_cast<T*>(out.value)[o] = none ? first : from_compute<T, typename cmp_of<T>::type>(st.best);
    }
}

// Feeds elements [lo, hi) of a dense row to `st`; `lane` of `lanes` cooperating threads.
// Whole 16-byte groups are fetched with one load, ragged edges element by element.
template <typename T, bool SUM, bool ARG, bool MIN>
__device__ __forceinline__ void scan_dense(State<T, SUM, ARG, MIN>& st, const T* row, int64_t lo, int64_t hi, int lane,
                                           int lanes) {
    constexpr int V = 16 / sizeof(T);
    const uintptr_t base = reinterpret_cast<uintptr_t>(row + lo);
    // element offset (relative to lo) of the first 16-byte boundary at or before row+lo
    const int64_t head = -static_cast<int64_t>((base & 15) / sizeof(T));
    const int64_t n = hi - lo;
    const int64_t stride = static_cast<int64_t>(lanes) * V;
    auto ragged = [&](int64_t g) {
#pragma unroll
        for (int k = 0; k < V; ++k) {
            const int64_t j = g + k;
            if (j >= 0 && j < n) st.feed(row[lo + j], lo + j);
        }
    };
    // Floating types with an index result: one strict comparison per 16-byte vector. The best of
    // the vector (fmax / fmin drop a NaN) is compared with a running extreme of its own and only the
    // vector's position is kept; the exact element is looked up once at the end and merged into the
    // state with the first-occurrence rule. Integers and sum-only scans feed element by element.
    using C = typename cmp_of<T>::type;
    using A = typename acc_of<T>::type;
    constexpr bool BY_VECTOR = ARG && (std::is_same<C, float>::value || std::is_same<C, double>::value);
    [[maybe_unused]] C vext = cmp_init<C, MIN>();
    [[maybe_unused]] int64_t vat = -1;
    auto feed_vector = [&](const T (&e)[V], int64_t at) {
        if constexpr (BY_VECTOR) {
            C m = to_compute<C>(e[0]);
            if constexpr (SUM) st.sum += to_compute<A>(e[0]);
#pragma unroll
            for (int k = 1; k < V; ++k) {
                const C v = to_compute<C>(e[k]);
                if constexpr (SUM) st.sum += to_compute<A>(e[k]);
                m = MIN ? fmin(m, v) : fmax(m, v);
            }
            if (MIN ? (m < vext) : (m > vext)) {
                vext = m;
                vat = at;
            }
        } else {
#pragma unroll
            for (int k = 0; k < V; ++k) st.feed(e[k], at + k);
        }
    };
    int64_t g = head + static_cast<int64_t>(lane) * V;
    if (g < 0) {  // only the lane that owns the group straddling the start of the range
        ragged(g);
        g += stride;
    }
    // four independent 16-byte loads in flight per lane
    for (; g + 3 * stride + V <= n; g += 4 * stride) {
        alignas(16) T e[4][V];
#pragma unroll
        for (int u = 0; u < 4; ++u) *reinterpret_cast<uint4*>(e[u]) = __ldg(reinterpret_cast<const uint4*>(row + lo + g + u * stride));
#pragma unroll
        for (int u = 0; u < 4; ++u) feed_vector(e[u], lo + g + u * stride);
    }
    for (; g + V <= n; g += stride) {
        alignas(16) T e[V];
        *reinterpret_cast<uint4*>(e) = __ldg(reinterpret_cast<const uint4*>(row + lo + g));
        feed_vector(e, lo + g);
    }
    if (g < n) ragged(g);
    if constexpr (BY_VECTOR) {
        if (vat >= 0) {
            alignas(16) T e[V];
            *reinterpret_cast<uint4*>(e) = __ldg(reinterpret_cast<const uint4*>(row + vat));
            int first = 0;
#pragma unroll
            for (int k = V - 1; k >= 0; --k)
                if (to_compute<C>(e[k]) == vext) first = k;  // equality: -0 and +0 tie, the lower index stays
            st.merge(A(0), to_compute<C>(e[first]), vat + first);  // the element itself keeps the sign of a zero
        }
    }
}

template <typename T, bool SUM, bool ARG, bool MIN>
__global__ void __launch_bounds__(kThreads) reduce_rows_warp(const T* __restrict__ src, int64_t rows, int64_t len, Outputs out) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * kThreads + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * kThreads) >> 5;
    for (int64_t r = warp; r < rows; r += nwarps) {
        const T* row = src + r * len;
        State<T, SUM, ARG, MIN> st;
        st.init();
        scan_dense(st, row, 0, len, lane, 32);
        warp_combine(st);
        if (lane == 0) write_out(st, out, r, len, len > 0 ? row[0] : T());
    }
}


// ---- one thread per row, rows staged per warp ---------------------------------------------
// Short rows of a 16-bit float type (up to 400 elements), dense source, last axis. A warp owns a span of
// 32 consecutive rows, which is one contiguous, 16-byte-aligned byte range: it copies the span into its own
// block of shared memory with coalesced 16-byte loads, then every lane reduces ONE row from there, so no
// partial results ever cross lanes. The row is read a word (two elements) at a time; per block of 16
// words a packed max / min tree gives the best even and the best odd element, compared (strictly, ordered:
// a NaN never wins, the first of equal values stays) with the row's running pair; only the block where
// each last improved is remembered and the element's position inside it is found by one scan at the end.
// Every warp has two blocks and copies its next span (cp.async) while it reduces the current one; up to
// 16 warps per CTA, one CTA per SM, and nothing but __syncwarp() orders anything.
constexpr int kLaneRows = 32;            // rows per span: one per lane
constexpr int kLaneMaxLen = 400;         // 2 blocks x 32 rows x 400 x 2 B = 50 KB per warp -> at least 4 warps per CTA
constexpr int kLaneSmemBytes = 200 << 10;

template <typename T, bool MIN> __device__ __forceinline__ uint32_t best_pair(uint32_t a, uint32_t b) {
    using T2 = typename pair_of_half<T>::type;
    const T2 m = MIN ? __hmin2(*reinterpret_cast<const T2*>(&a), *reinterpret_cast<const T2*>(&b))
                     : __hmax2(*reinterpret_cast<const T2*>(&a), *reinterpret_cast<const T2*>(&b));
    return *reinterpret_cast<const uint32_t*>(&m);
}

template <typename T, bool SUM, bool ARG, bool MIN>
__global__ void __launch_bounds__(512, 1) reduce_rows_lane(const T* __restrict__ src, int64_t rows, int len, uint32_t span_stride,
                                                           Outputs out) {
    static_assert(sizeof(T) == 2, "16-bit float types only");
    extern __shared__ __align__(128) unsigned char lane_smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    // two blocks per warp: the copy of the warp's next span runs while the current one is reduced
    unsigned char* blocks = lane_smem + static_cast<size_t>(warp) * 2 * span_stride;
    const int64_t spans = (rows + kLaneRows - 1) / kLaneRows;
    const uint32_t none = pair_bits<T>(cmp_init<float, MIN>());
    const int64_t step = static_cast<int64_t>(gridDim.x) * warps;
    auto fetch = [&](int64_t span, unsigned char* stage) {
        if (span < spans) {
            const int64_t row0 = span * kLaneRows;
            const int nrows = static_cast<int>(rows - row0 < kLaneRows ? rows - row0 : kLaneRows);
            const int elems = nrows * len;
            const unsigned char* g = reinterpret_cast<const unsigned char*>(src + row0 * len);  // 64 * len bytes per span: 16-byte aligned
            const int vecs = (elems * 2) >> 4;
            const uint32_t sbase = static_cast<uint32_t>(__cvta_generic_to_shared(stage));
            for (int v = lane; v < vecs; v += 32)
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sbase + v * 16), "l"(g + static_cast<size_t>(v) * 16) : "memory");
            for (int e = vecs * 8 + lane; e < elems; e += 32)  // ragged end of the last span
                reinterpret_cast<uint16_t*>(stage)[e] = reinterpret_cast<const uint16_t*>(g)[e];
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    int which = 0;
    int64_t span = static_cast<int64_t>(blockIdx.x) * warps + warp;
    fetch(span, blocks);
    for (; span < spans; span += step, which ^= 1) {
        unsigned char* stage = blocks + static_cast<size_t>(which) * span_stride;
        fetch(span + step, blocks + static_cast<size_t>(which ^ 1) * span_stride);  // the other block was released by the __syncwarp that ended the last pass
        asm volatile("cp.async.wait_group 1;" ::: "memory");                      // all but the newest group have landed
        __syncwarp();
        const int64_t row0 = span * kLaneRows;
        const int nrows = static_cast<int>(rows - row0 < kLaneRows ? rows - row0 : kLaneRows);
        if (lane < nrows) {
            const T* row = reinterpret_cast<const T*>(stage) + lane * len;
            const int odd = (lane * len) & 1;  // the row starts in the upper half of a word: peel one element
            const uint32_t* words = reinterpret_cast<const uint32_t*>(row + odd);
            const int nwords = (len - odd) >> 1;
            State<T, SUM, ARG, MIN> st;
            st.init();
            if (odd) st.feed(row[0], 0);
            float sum_lo = 0.0f, sum_hi = 0.0f;
            float best_lo = cmp_init<float, MIN>(), best_hi = cmp_init<float, MIN>();
            int block_lo = -1, block_hi = -1;
            for (int b0 = 0; b0 < nwords; b0 += 16) {
                uint32_t m = none;
                if (b0 + 16 <= nwords) {
                    uint32_t w[16];
#pragma unroll
                    for (int k = 0; k < 16; ++k) w[k] = words[b0 + k];
                    if constexpr (ARG) {
                        uint32_t t8[8];
#pragma unroll
                        for (int k = 0; k < 8; ++k) t8[k] = best_pair<T, MIN>(w[k], w[k + 8]);
#pragma unroll
                        for (int k = 0; k < 4; ++k) t8[k] = best_pair<T, MIN>(t8[k], t8[k + 4]);
                        m = best_pair<T, MIN>(best_pair<T, MIN>(t8[0], t8[2]), best_pair<T, MIN>(t8[1], t8[3]));
                    }
                    if constexpr (SUM) {
#pragma unroll
                        for (int k = 0; k < 16; ++k) {
                            sum_lo += half_of_pair<T>(w[k], 0);
                            sum_hi += half_of_pair<T>(w[k], 1);
                        }
                    }
                } else {
                    for (int k = b0; k < nwords; ++k) {
                        const uint32_t w = words[k];
                        if constexpr (ARG) m = best_pair<T, MIN>(m, w);
                        if constexpr (SUM) {
                            sum_lo += half_of_pair<T>(w, 0);
                            sum_hi += half_of_pair<T>(w, 1);
                        }
                    }
                }
                if constexpr (ARG) {
                    const float lo = half_of_pair<T>(m, 0), hi = half_of_pair<T>(m, 1);
                    if (MIN ? (lo < best_lo) : (lo > best_lo)) {
                        best_lo = lo;
                        block_lo = b0;
                    }
                    if (MIN ? (hi < best_hi) : (hi > best_hi)) {
                        best_hi = hi;
                        block_hi = b0;
                    }
                }
            }
            if constexpr (SUM) st.sum += sum_lo + sum_hi;
            if constexpr (ARG) {
                // position of each half's extreme inside the block where it first appeared
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int b0 = h ? block_hi : block_lo;
                    const float best = h ? best_hi : best_lo;
                    if (b0 >= 0) {
                        int at = 0;
                        const int top = nwords - b0 < 16 ? nwords - b0 : 16;
#pragma unroll 4
                        for (int k = 15; k >= 0; --k)
                            if (k < top && half_of_pair<T>(words[b0 + k], h) == best) at = k;
                        const int j = odd + 2 * (b0 + at) + h;
                        st.merge(0.0f, to_compute<float>(row[j]), j);  // the element itself: the sign of a zero survives
                    }
                }
            }
            if ((len - odd) & 1) {
                State<T, SUM, ARG, MIN> tail;
                tail.init();
                tail.feed(row[len - 1], len - 1);
                st.merge(tail);
            }
            write_out(st, out, row0 + lane, len, row[0]);
        }
        __syncwarp();  // every lane is done with the block before the next span overwrites it
    }
}

// ---- staged short rows -------------------------------------------------------------------
constexpr int kStagedThreads = 512;

__device__ unsigned int g_reduce_aborts = 0;  // no bounded waits remain in this file; kept for the error counter

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

// rows_per_chunk rows of `len` elements are contiguous in memory; chunk k starts at row
// k * rows_per_chunk. A chunk (a multiple of 16 bytes, 16-byte aligned because rows_per_chunk is a
// multiple of 16) is brought into shared memory with per-thread 16-byte asynchronous copies
// (cp.async), double-buffered: the copy of the next chunk is in flight while the current one is
// reduced. (A single TMA bulk copy per chunk was measured at 3.9 TB/s at best; the per-thread
// copies keep many more requests in flight.) The ragged last chunk uses ordinary loads.
// `lanes` (a power of two <= 32) threads share a row: lane q visits elements q, q + lanes, ...
// in ascending order and the partial results are merged with shuffles (lowest index wins ties).
template <typename T, bool SUM, bool ARG, bool MIN, bool PAD>
__global__ void __launch_bounds__(kStagedThreads) reduce_rows_staged(const T* __restrict__ src, int64_t rows, int len,
                                                                    int rows_per_chunk, int lanes, Outputs out) {
    constexpr bool padded = PAD;
    // PAD (rows that are a multiple of 16 bytes): every staged row gets 16 bytes of padding
    // and is read with 16-byte loads, which keeps rows of 64, 128, ... bytes off the same banks
    extern __shared__ __align__(128) unsigned char staged_smem[];
    using A = typename acc_of<T>::type;
    using C = typename cmp_of<T>::type;
    const uint32_t row_bytes = static_cast<uint32_t>(len) * sizeof(T);
    const uint32_t pitch = padded ? row_bytes + 16u : row_bytes;
    const uint32_t vectors_per_row = row_bytes >> 4;
    const uint32_t chunk_bytes = static_cast<uint32_t>(rows_per_chunk) * row_bytes;
    const uint32_t buf_stride = (static_cast<uint32_t>(rows_per_chunk) * pitch + 127u) & ~127u;
    auto buffer = [&](int b) { return reinterpret_cast<T*>(staged_smem + static_cast<size_t>(b) * buf_stride); };
    const int64_t chunks = (rows + rows_per_chunk - 1) / rows_per_chunk;
    const uint32_t vectors = chunk_bytes >> 4;
    auto issue = [&](int64_t chunk, int b) {
        // every thread starts its share of the 16-byte copies of a full chunk, then closes the group
        const int64_t first = chunk * rows_per_chunk;
        if (chunk < chunks && first + rows_per_chunk <= rows) {
            const unsigned char* g = reinterpret_cast<const unsigned char*>(src + first * len);
            const uint32_t sbase = smem_addr(buffer(b));
            for (uint32_t v = threadIdx.x; v < vectors; v += blockDim.x) {
                uint32_t dst = v * 16;
                if constexpr (PAD) dst += (v / vectors_per_row) * 16;  // one pad per completed row
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sbase + dst), "l"(g + static_cast<size_t>(v) * 16) : "memory");
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    int b = 0;
    int64_t chunk = blockIdx.x;
    issue(chunk, 0);
    for (; chunk < chunks; chunk += gridDim.x, b ^= 1) {
        issue(chunk + gridDim.x, b ^ 1);  // the other buffer was released by the barrier that ended the last pass
        const int64_t first = chunk * rows_per_chunk;
        const bool full = first + rows_per_chunk <= rows;
        const int here = static_cast<int>(full ? rows_per_chunk : rows - first);
        if (full) {
            asm volatile("cp.async.wait_group 1;" ::: "memory");  // all but the newest group have landed
        } else {
            const int64_t n = static_cast<int64_t>(here) * len;
            const int pad_elems = padded ? static_cast<int>(16 / sizeof(T)) : 0;
            for (int64_t i = threadIdx.x; i < n; i += blockDim.x) buffer(b)[i + (i / len) * pad_elems] = src[first * len + i];
        }
        __syncthreads();
        {
            const int r = static_cast<int>(threadIdx.x) / lanes, q = static_cast<int>(threadIdx.x) % lanes;
            const bool active = r < here;
            const T* row = reinterpret_cast<const T*>(reinterpret_cast<const unsigned char*>(buffer(b)) + static_cast<size_t>(active ? r : 0) * pitch);
            A sum = A(0);
            C best = cmp_init<C, MIN>();
            int idx = INT_MAX;
            auto feed = [&](T raw, int j, A& acc) {
                if constexpr (SUM) acc += to_compute<A>(raw);
                if constexpr (ARG) {
                    const C v = to_compute<C>(raw);
                    if (MIN ? (v < best) : (v > best)) { best = v; idx = j; }
                }
            };
            if constexpr (PAD) {
              if (active) {
                // 16-byte vectors, dealt to the row's lanes in turn: ascending indices per lane
                constexpr int PER = 16 / static_cast<int>(sizeof(T));
                const uint4* vecs = reinterpret_cast<const uint4*>(row);
                if constexpr (ARG && (std::is_same<C, float>::value || std::is_same<C, double>::value)) {
                    // floating types: one strict comparison per vector, the element settled afterwards
                    C ext = cmp_init<C, MIN>();
                    int at = -1;
#pragma unroll 2
                    for (int c = q; c < static_cast<int>(vectors_per_row); c += lanes) {
                        const uint4 v = vecs[c];
                        const T* e = reinterpret_cast<const T*>(&v);
                        C m = to_compute<C>(e[0]);
                        if constexpr (SUM) sum += to_compute<A>(e[0]);
#pragma unroll
                        for (int k = 1; k < PER; ++k) {
                            const C x = to_compute<C>(e[k]);
                            if constexpr (SUM) sum += to_compute<A>(e[k]);
                            m = MIN ? fmin(m, x) : fmax(m, x);
                        }
                        if (MIN ? (m < ext) : (m > ext)) {
                            ext = m;
                            at = c;
                        }
                    }
                    if (at >= 0) {
                        const uint4 v = vecs[at];
                        const T* e = reinterpret_cast<const T*>(&v);
                        int first = 0;
#pragma unroll
                        for (int k = PER - 1; k >= 0; --k)
                            if (to_compute<C>(e[k]) == ext) first = k;
                        best = ext;
                        idx = at * PER + first;
                    }
                } else {
#pragma unroll 2
                    for (int c = q; c < static_cast<int>(vectors_per_row); c += lanes) {
                        const uint4 v = vecs[c];
                        const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
                        for (int k = 0; k < PER; ++k) feed(e[k], c * PER + k, sum);
                    }
                }
              }
            } else if (active) {
                if constexpr (sizeof(T) == 2) {
                    // 16-bit elements are read two at a time as 32-bit words. A row that starts on an
                    // odd element is peeled by one; lane 0 takes the peeled head and a leftover tail,
                    // so every lane still meets its indices in ascending order.
                    const int off = static_cast<int>((reinterpret_cast<uintptr_t>(row) >> 1) & 1);
                    const int npairs = (len - off) >> 1;
                    const uint32_t* words = reinterpret_cast<const uint32_t*>(row + off);
                    A sum_hi = A(0);
                    if (off && q == 0) feed(row[0], 0, sum);
                    if constexpr (ARG && is_half16<T>::value) {
                        // Floats: both halves of a word are compared at once with packed 16-bit
                        // arithmetic. Each half keeps a running extreme and the (16-bit) word position
                        // where it last improved; a strict ordered comparison never selects a NaN and
                        // keeps the first of equal values. The two halves are merged once, afterwards.
                        using T2 = typename pair_of_half<T>::type;
                        uint32_t run = pair_bits<T>(cmp_init<float, MIN>());
                        uint32_t at2 = 0xFFFFFFFFu;                       // 0xFFFF: this half never improved
                        uint32_t pr2 = static_cast<uint32_t>(q) * 0x00010001u;
                        const uint32_t step2 = static_cast<uint32_t>(lanes) * 0x00010001u;
#pragma unroll 4
                        for (int pr = q; pr < npairs; pr += lanes, pr2 += step2) {
                            const uint32_t w = words[pr];
                            if constexpr (SUM) {
                                sum += half_of_pair<T>(w, 0);
                                sum_hi += half_of_pair<T>(w, 1);
                            }
                            const T2 x = *reinterpret_cast<const T2*>(&w), r2 = *reinterpret_cast<const T2*>(&run);
                            const uint32_t better = MIN ? __hlt2_mask(x, r2) : __hgt2_mask(x, r2);
                            run = (w & better) | (run & ~better);
                            at2 = (pr2 & better) | (at2 & ~better);
                        }
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const uint32_t at = (at2 >> (16 * h)) & 0xFFFFu;
                            if (at != 0xFFFFu) {
                                const float v = half_of_pair<T>(run, h);
                                const int j = off + 2 * static_cast<int>(at) + h;
                                if ((MIN ? (v < best) : (v > best)) || (v == best && j < idx)) {
                                    best = v;
                                    idx = j;
                                }
                            }
                        }
                    } else {
#pragma unroll 4
                        for (int pr = q; pr < npairs; pr += lanes) {
                            const uint32_t w = words[pr];
                            const uint16_t lo = static_cast<uint16_t>(w & 0xffffu), hi = static_cast<uint16_t>(w >> 16);
                            feed(*reinterpret_cast<const T*>(&lo), off + 2 * pr, sum);
                            feed(*reinterpret_cast<const T*>(&hi), off + 2 * pr + 1, sum_hi);
                        }
                    }
                    if (((len - off) & 1) && q == 0) feed(row[len - 1], len - 1, sum);
                    if constexpr (SUM) sum += sum_hi;
                } else {
#pragma unroll 4
                    for (int j = q; j < len; j += lanes) feed(row[j], j, sum);
                }
            }
            // rows never straddle a warp (lanes divides 32): merge the lanes of a row
            for (int m = lanes >> 1; m > 0; m >>= 1) {
                if constexpr (SUM) sum += shfl_xor(sum, m);
                if constexpr (ARG) {
                    const C ob = shfl_xor(best, m);
                    const int oi = __shfl_xor_sync(0xffffffffu, idx, m);
                    if ((MIN ? (ob < best) : (ob > best)) || (ob == best && oi < idx)) { best = ob; idx = oi; }
                }
            }
            if (active && q == 0) {
                const int64_t o = first + r;
                if constexpr (SUM) {
                    if (out.sum) static_cast<T*>(out.sum)[o] = from_compute<T, A>(out.mean ? sum / static_cast<A>(len) : sum);
                }
                if constexpr (ARG) {
                    if (out.index) out.index[o] = idx == INT_MAX ? 0 : idx;
                    if (out.value) static_cast<T*>(out.value)[o] = row[idx == INT_MAX ? 0 : idx];  // the element itself (keeps the sign of a zero)
                }
            }
        }
        __syncthreads();  // everyone is done with buffer b before it is refilled two passes on
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
}

template <typename T, bool SUM, bool ARG, bool MIN>
__device__ __forceinline__ void block_combine(State<T, SUM, ARG, MIN>& st) {
    using S = State<T, SUM, ARG, MIN>;
    __shared__ typename S::A s_sum[kThreads / 32];
    __shared__ typename S::C s_best[kThreads / 32];
    __shared__ int64_t s_idx[kThreads / 32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    warp_combine(st);
    __syncthreads();  // protects the arrays across successive calls
    if (lane == 0) {
        s_sum[warp] = st.sum;
        s_best[warp] = st.best;
        s_idx[warp] = st.idx;
    }
    __syncthreads();
    if (warp == 0) {
        if (lane < kThreads / 32) {
            st.sum = s_sum[lane];
            st.best = s_best[lane];
            st.idx = s_idx[lane];
        } else {
            st.init();
        }
        warp_combine(st);
    }
}

template <typename T, bool SUM, bool ARG, bool MIN>
__global__ void __launch_bounds__(kThreads) reduce_rows_block(const T* __restrict__ src, int64_t rows, int64_t len, Outputs out) {
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const T* row = src + r * len;
        State<T, SUM, ARG, MIN> st;
        st.init();
        scan_dense(st, row, 0, len, threadIdx.x, kThreads);
        block_combine(st);
        if (threadIdx.x == 0) write_out(st, out, r, len, len > 0 ? row[0] : T());
    }
}

// Partial result of one segment of one row, kept in scratch memory between the two kernels of
// the split reduction.
template <typename T> struct Partial {
    typename acc_of<T>::type sum;
    typename cmp_of<T>::type best;
    int64_t idx;
};

template <typename T, bool SUM, bool ARG, bool MIN>
__global__ void __launch_bounds__(kThreads) reduce_split_partial(const T* __restrict__ src, int64_t len, int splits,
                                                                 Partial<T>* __restrict__ scratch) {
    const int64_t r = blockIdx.y;
    const int seg = blockIdx.x;
    const int64_t per = (len + splits - 1) / splits;
    const int64_t lo = (int64_t)seg * per;
    const int64_t hi = lo + per < len ? lo + per : len;
    State<T, SUM, ARG, MIN> st;
    st.init();
    if (lo < hi) scan_dense(st, src + r * len, lo, hi, threadIdx.x, kThreads);
    block_combine(st);
    if (threadIdx.x == 0) {
        Partial<T> p;
        p.sum = st.sum;
        p.best = st.best;
        p.idx = st.idx;
        scratch[r * splits + seg] = p;
    }
}

template <typename T, bool SUM, bool ARG, bool MIN>
__global__ void __launch_bounds__(32) reduce_split_final(const T* __restrict__ src, int64_t rows, int64_t len, int splits,
                                                         const Partial<T>* __restrict__ scratch, Outputs out) {
    const int64_t r = blockIdx.x;
    if (r >= rows) return;
    State<T, SUM, ARG, MIN> st;
    st.init();
    // segments are visited in ascending order per lane and merged with the lowest-index rule
    for (int s = threadIdx.x; s < splits; s += 32) {
        const Partial<T> p = scratch[r * splits + s];
        st.merge(p.sum, p.best, p.idx);
    }
    warp_combine(st);
    if (threadIdx.x == 0) write_out(st, out, r, len, len > 0 ? src[r * len] : T());
}

// Source dense as [outer, len, inner]; thread per (outer, inner) output.
template <typename T, bool SUM, bool ARG, bool MIN>
__global__ void __launch_bounds__(kThreads) reduce_cols(const T* __restrict__ src, int64_t outer, int64_t len, int64_t inner,
                                                        Outputs out) {
    const int64_t total = outer * inner;
    const int64_t step = (int64_t)gridDim.x * kThreads;
    for (int64_t o = (int64_t)blockIdx.x * kThreads + threadIdx.x; o < total; o += step) {
        const int64_t ou = o / inner, in = o - ou * inner;
        const T* col = src + ou * len * inner + in;
        State<T, SUM, ARG, MIN> st;
        st.init();
        int64_t l = 0;
        for (; l + 4 <= len; l += 4) {
            T v0 = __ldg(col + (l + 0) * inner), v1 = __ldg(col + (l + 1) * inner);
            T v2 = __ldg(col + (l + 2) * inner), v3 = __ldg(col + (l + 3) * inner);
            st.feed(v0, l);
            st.feed(v1, l + 1);
            st.feed(v2, l + 2);
            st.feed(v3, l + 3);
        }
        for (; l < len; ++l) st.feed(__ldg(col + l * inner), l);
        write_out(st, out, o, len, len > 0 ? col[0] : T());
    }
}

// ---- inner-axis reduction of a dense [outer, len, inner] tensor ---------------------------
// A CTA is 32 x 8 threads: x runs along `inner` (VEC consecutive outputs per thread, one 16-byte
// load when VEC > 1), y splits the reduced axis inside the CTA, blockIdx.z splits it across CTAs.
// The eight y-partials are merged through shared memory; with more than one z-split the CTA result
// goes to scratch memory as a Partial and reduce_cols_final merges the splits in ascending order.
template <typename T, bool SUM, bool ARG, bool MIN, int VEC>
__global__ void __launch_bounds__(256) reduce_cols_tiled(const T* __restrict__ src, int64_t len, int64_t inner, int64_t chunk,
                                                        Partial<T>* __restrict__ scratch, Outputs out) {
    using S = State<T, SUM, ARG, MIN>;
    __shared__ typename S::A s_sum[8][33];
    __shared__ typename S::C s_best[8][33];
    __shared__ int64_t s_idx[8][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int64_t col0 = (static_cast<int64_t>(blockIdx.x) * 32 + tx) * VEC;
    const int64_t ou = blockIdx.y;
    const int64_t l0 = static_cast<int64_t>(blockIdx.z) * chunk;
    const int64_t l1 = l0 + chunk < len ? l0 + chunk : len;
    const bool in_range = col0 < inner;
    S st[VEC];
#pragma unroll
    for (int k = 0; k < VEC; ++k) st[k].init();
    if (in_range) {
        const T* base = src + ou * len * inner + col0;
        int64_t l = l0 + ty;
        // four rows in flight per thread (64 bytes): with six CTAs resident per SM that is about 96 KiB
        // of loads in flight per SM, enough to cover the HBM latency
        for (; l + 24 < l1; l += 32) {
            alignas(16) T e[4][VEC];
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                if constexpr (VEC > 1) *reinterpret_cast<uint4*>(e[r]) = __ldg(reinterpret_cast<const uint4*>(base + (l + 8 * r) * inner));
                else e[r][0] = __ldg(base + (l + 8 * r) * inner);
            }
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int k = 0; k < VEC; ++k) st[k].feed(e[r][k], l + 8 * r);
        }
        for (; l < l1; l += 8) {
            alignas(16) T e0[VEC];
            if constexpr (VEC > 1) *reinterpret_cast<uint4*>(e0) = __ldg(reinterpret_cast<const uint4*>(base + l * inner));
            else e0[0] = __ldg(base + l * inner);
#pragma unroll
            for (int k = 0; k < VEC; ++k) st[k].feed(e0[k], l);
        }
    }
    const int64_t total = static_cast<int64_t>(gridDim.y) * inner;
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
        __syncthreads();
        s_sum[ty][tx] = st[k].sum;
        s_best[ty][tx] = st[k].best;
        s_idx[ty][tx] = st[k].idx;
        __syncthreads();
        if (ty == 0 && in_range && col0 + k < inner) {
            S acc = st[k];
            for (int y = 1; y < 8; ++y) acc.merge(s_sum[y][tx], s_best[y][tx], s_idx[y][tx]);
            const int64_t o = ou * inner + col0 + k;
            if (scratch != nullptr) {
                Partial<T> p;
                p.sum = acc.sum;
                p.best = acc.best;
                p.idx = acc.idx;
                scratch[static_cast<int64_t>(blockIdx.z) * total + o] = p;
            } else {
                write_out(acc, out, o, len, len > 0 ? src[ou * len * inner + col0 + k] : T());
            }
        }
    }
}

template <typename T, bool SUM, bool ARG, bool MIN>
__global__ void __launch_bounds__(kThreads) reduce_cols_final(const T* __restrict__ src, int64_t total, int64_t len, int64_t inner,
                                                              int splits, const Partial<T>* __restrict__ scratch, Outputs out) {
    const int64_t o = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
    if (o >= total) return;
    State<T, SUM, ARG, MIN> st;
    st.init();
    for (int z = 0; z < splits; ++z) {
        const Partial<T> p = scratch[static_cast<int64_t>(z) * total + o];
        st.merge(p.sum, p.best, p.idx);
    }
    const int64_t ou = o / inner, in = o - ou * inner;
    write_out(st, out, o, len, len > 0 ? src[ou * len * inner + in] : T());
}

struct StridedGeom {
    int rank;                     // dims other than the axis
    int64_t sizes[TN_MAX_RANK];   // their extents, outermost first
    int64_t strides[TN_MAX_RANK]; // their element strides
    int64_t len, axis_stride, total;
};

template <typename T, bool SUM, bool ARG, bool MIN>
__global__ void __launch_bounds__(kThreads) reduce_strided(const T* __restrict__ src, StridedGeom g, Outputs out) {
    const int64_t step = (int64_t)gridDim.x * kThreads;
    for (int64_t o = (int64_t)blockIdx.x * kThreads + threadIdx.x; o < g.total; o += step) {
        int64_t rem = o, off = 0;
        for (int d = g.rank - 1; d >= 0; --d) {
            const int64_t c = rem % g.sizes[d];
            rem /= g.sizes[d];
            off += c * g.strides[d];
        }
        State<T, SUM, ARG, MIN> st;
        st.init();
        for (int64_t l = 0; l < g.len; ++l) st.feed(src[off + l * g.axis_stride], l);
        write_out(st, out, o, g.len, g.len > 0 ? src[off] : T());
    }
}

// ------------------------------------------------------------------ host --------------
int64_t env_int64(const char* name, int64_t fallback) { return env_knob(name, (int)fallback); }

int grid_cap() { return sm_count() * 8; }

// Launch of the staged kernel. TN_UNSUPPORTED_DTYPE means "rows too long for a chunk" and sends
// the caller on to the next kernel; it is never returned to the user from here.
template <typename T, bool SUM, bool ARG, bool MIN, bool PAD>
tn_status launch_staged(const T* p, int64_t total, int64_t len, int chunk_kb, Outputs out, cudaStream_t s) {
    const int64_t row_bytes = len * (int64_t)sizeof(T);
    const int64_t pitch = row_bytes + (PAD ? 16 : 0);
    // threads per row: about 64 elements and up per thread. Fewer, longer scans measured
    // faster than wide ones (197-wide bf16 rows: 2 threads per row 3.97 TB/s, 4 or 8: 3.48)
    int lanes = 1;
    while (lanes < 8 && len >= 128 * lanes) lanes *= 2;
    if (const int n = env_knob("TN_REDUCE_LANES", 0); n == 1 || n == 2 || n == 4 || n == 8) lanes = n;
    int rpc = (int)((int64_t(chunk_kb) << 10) / pitch);
    if (rpc > kStagedThreads / lanes) rpc = kStagedThreads / lanes;
    rpc &= ~15;  // a chunk of 16 rows is a multiple of 16 bytes for any row length
    if (rpc < 16) return TN_UNSUPPORTED_DTYPE;
    const int threads = (rpc * lanes + 31) & ~31;  // one group of `lanes` threads per row of a chunk
    const size_t buf = ((size_t)rpc * pitch + 127) & ~size_t(127);
    const size_t smem = 2 * buf;
    static thread_local int attr_device = -1;
    int dev = 0;
    TN_CUDA(cudaGetDevice(&dev));
    if (attr_device != dev) {
        TN_CUDA(cudaFuncSetAttribute(reduce_rows_staged<T, SUM, ARG, MIN, PAD>, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 << 10));
        attr_device = dev;
    }
    const int64_t chunks = ceil_div(total, rpc);
    int64_t per_sm = (int64_t(220) << 10) / (int64_t)smem;  // CTAs that fit the shared memory of an SM
    if (per_sm > 2048 / threads) per_sm = 2048 / threads;
    if (per_sm > 16) per_sm = 16;
    if (per_sm < 1) per_sm = 1;
    int64_t grid = (int64_t)sm_count() * per_sm;
    if (grid > chunks) grid = chunks;
    reduce_rows_staged<T, SUM, ARG, MIN, PAD><<<(unsigned)grid, threads, smem, s>>>(p, total, (int)len, rpc, lanes, out);
    return after_launch("reduce_rows_staged");
}

template <typename T, bool SUM, bool ARG, bool MIN>
tn_status launch(const tn_tensor_t* src, int axis, Outputs out, cudaStream_t s) {
    const int R = src->rank;
    int64_t outer = 1, inner = 1;
    const int64_t len = (int64_t)src->shape.sizes[axis];
    for (int d = 0; d < axis; ++d) outer *= (int64_t)src->shape.sizes[d];
    for (int d = axis + 1; d < R; ++d) inner *= (int64_t)src->shape.sizes[d];
    const int64_t total = outer * inner;
    if (total == 0) return TN_SUCCESS;
    // dense row-major?
    bool dense = true;
    int64_t expect = 1;
    for (int d = R - 1; d >= 0; --d) {
        const int64_t sz = (int64_t)src->shape.sizes[d];
        if (sz != 1 && src->strides.sizes[d] != expect) dense = false;
        expect *= sz;
    }
    const T* p = static_cast<const T*>(src->address);
    const int cap = grid_cap();
    if (dense && inner == 1) {
        const int64_t row_bytes = len * (int64_t)sizeof(T);
        if (total < (int64_t)sm_count() && row_bytes >= (int64_t(1) << 20)) {
            // few very long rows: cut each into segments so every SM streams a share
            int splits = (int)ceil_div((int64_t)sm_count() * 4, total);
            const int64_t max_splits = ceil_div(row_bytes, int64_t(64) << 10);
            if (splits > max_splits) splits = (int)max_splits;
            if (splits > 1024) splits = 1024;
            Partial<T>* scratch = nullptr;
            TN_TRY(scratch_alloc(reinterpret_cast<void**>(&scratch), sizeof(Partial<T>) * total * splits, s));
            reduce_split_partial<T, SUM, ARG, MIN><<<dim3(splits, (unsigned)total), kThreads, 0, s>>>(p, len, splits, scratch);
            tn_status st = after_launch("reduce_split_partial");
            if (st == TN_SUCCESS) {
                reduce_split_final<T, SUM, ARG, MIN><<<(unsigned)total, 32, 0, s>>>(p, total, len, splits, scratch, out);
                st = after_launch("reduce_split_final");
            }
            tn_status fr = scratch_free(scratch, s);
            return st != TN_SUCCESS ? st : fr;
        }
        // 16-bit floats, rows of up to 400 elements, many rows: one thread per row on warp-private staged spans
        if constexpr (is_half16<T>::value) {
            static const bool no_lane = getenv("TN_REDUCE_NO_LANE") != nullptr;
            if (!no_lane && len >= 8 && len <= kLaneMaxLen && total >= 4096 && (reinterpret_cast<uintptr_t>(p) & 15) == 0) {
                const uint32_t span_stride = (uint32_t)((kLaneRows * len * 2 + 127) & ~int64_t(127));
                int warps = (int)(kLaneSmemBytes / (2 * span_stride));
                if (warps > 16) warps = 16;
                const size_t smem = (size_t)warps * 2 * span_stride;
                static thread_local int attr_device = -1;
                int dev = 0;
                TN_CUDA(cudaGetDevice(&dev));
                if (attr_device != dev) {
                    TN_CUDA(cudaFuncSetAttribute(reduce_rows_lane<T, SUM, ARG, MIN>, cudaFuncAttributeMaxDynamicSharedMemorySize, kLaneSmemBytes));
                    attr_device = dev;
                }
                const int64_t spans = ceil_div(total, kLaneRows);
                int64_t grid = ceil_div(spans, warps);
                if (grid > sm_count()) grid = sm_count();
                reduce_rows_lane<T, SUM, ARG, MIN><<<(unsigned)grid, warps * 32, smem, s>>>(p, total, (int)len, span_stride, out);
                return after_launch("reduce_rows_lane");
            }
        }
        // Rows up to 1 KiB always take the staged kernel; up to 2 KiB they do unless the row is a
        // whole number of 512-byte warp sweeps, where the warp-per-row kernel is balanced and measured
        // faster (768 fp16: 5.4 against 3.8 TB/s; 1000 bf16 the other way round: 3.7 against 5.0 TB/s).
        static const int64_t staged_max = env_int64("TN_REDUCE_STAGED_MAX_BYTES", 2048);
        const bool staged_fits = row_bytes <= 1024 || (row_bytes <= staged_max && row_bytes % 512 != 0);
        if (staged_fits && len >= 8 && total >= 2048 && (reinterpret_cast<uintptr_t>(p) & 15) == 0) {
            // whole rows staged in shared memory: rows per chunk is a multiple of 16 so that a
            // chunk is a multiple of 16 bytes for any row length
            int chunk_kb = 50;
            if (const int n = env_knob("TN_REDUCE_CHUNK_KB", 0); n >= 4 && n <= 52) chunk_kb = n;
            const bool padded = row_bytes % 16 == 0;
            tn_status st = padded ? launch_staged<T, SUM, ARG, MIN, true>(p, total, len, chunk_kb, out, s)
                                  : launch_staged<T, SUM, ARG, MIN, false>(p, total, len, chunk_kb, out, s);
            if (st != TN_UNSUPPORTED_DTYPE) return st;  // else: the rows do not fit this kernel, fall through
        }
        if (row_bytes >= 16384) {
            const int grid = (int)(total < cap ? total : cap);
            reduce_rows_block<T, SUM, ARG, MIN><<<grid, kThreads, 0, s>>>(p, total, len, out);
            return after_launch("reduce_rows_block");
        }
        int64_t blocks = ceil_div(total, kThreads / 32);
        if (blocks > cap) blocks = cap;
        reduce_rows_warp<T, SUM, ARG, MIN><<<(int)blocks, kThreads, 0, s>>>(p, total, len, out);
        return after_launch("reduce_rows_warp");
    }
    if (dense && inner >= 32 && outer <= 65535) {
        constexpr int V = 16 / (int)sizeof(T);
        const bool vec = V > 1 && inner % V == 0 && (reinterpret_cast<uintptr_t>(p) & 15) == 0;
        const int64_t per_thread = vec ? V : 1;
        const int64_t gx = ceil_div(inner, 32 * per_thread);
        // split the reduced axis across CTAs until about six CTAs per SM exist
        int64_t splits = ceil_div((int64_t)sm_count() * env_knob("TN_REDUCE_COLS_CTAS_PER_SM", 6), gx * outer);
        if (splits > len / 64) splits = len / 64;
        if (splits < 1) splits = 1;
        if (splits > 1024) splits = 1024;
        const int64_t chunk = ceil_div(len, splits);
        splits = ceil_div(len, chunk);
        Partial<T>* scratch = nullptr;
        if (splits > 1) TN_TRY(scratch_alloc(reinterpret_cast<void**>(&scratch), sizeof(Partial<T>) * total * splits, s));
        const dim3 grid((unsigned)gx, (unsigned)outer, (unsigned)splits);
        if (vec) reduce_cols_tiled<T, SUM, ARG, MIN, V><<<grid, 256, 0, s>>>(p, len, inner, chunk, scratch, out);
        else reduce_cols_tiled<T, SUM, ARG, MIN, 1><<<grid, 256, 0, s>>>(p, len, inner, chunk, scratch, out);
        tn_status st = after_launch("reduce_cols_tiled");
        if (splits > 1) {
            if (st == TN_SUCCESS) {
                reduce_cols_final<T, SUM, ARG, MIN><<<(unsigned)ceil_div(total, kThreads), kThreads, 0, s>>>(p, total, len, inner, (int)splits, scratch, out);
                st = after_launch("reduce_cols_final");
            }
            const tn_status fr = scratch_free(scratch, s);
            if (st == TN_SUCCESS) st = fr;
        }
        return st;
    }
    if (dense) {
        int64_t blocks = ceil_div(total, kThreads);
        if (blocks > cap) blocks = cap;
        reduce_cols<T, SUM, ARG, MIN><<<(int)blocks, kThreads, 0, s>>>(p, outer, len, inner, out);
        return after_launch("reduce_cols");
    }
    StridedGeom g;
    g.rank = 0;
    for (int d = 0; d < R; ++d) {
        if (d == axis) continue;
        g.sizes[g.rank] = (int64_t)src->shape.sizes[d];
        g.strides[g.rank] = src->strides.sizes[d];
        ++g.rank;
    }
    g.len = len;
    g.axis_stride = src->strides.sizes[axis];
    g.total = total;
    int64_t blocks = ceil_div(total, kThreads);
    if (blocks > cap) blocks = cap;
    reduce_strided<T, SUM, ARG, MIN><<<(int)blocks, kThreads, 0, s>>>(p, g, out);
    return after_launch("reduce_strided");
}

template <bool SUM, bool ARG, bool MIN>
tn_status by_dtype(const tn_tensor_t* src, int axis, Outputs out, cudaStream_t s) {
    switch (src->dtype) {
        case TN_INT8: return launch<int8_t, SUM, ARG, MIN>(src, axis, out, s);
        case TN_INT16: return launch<int16_t, SUM, ARG, MIN>(src, axis, out, s);
        case TN_INT32: return launch<int32_t, SUM, ARG, MIN>(src, axis, out, s);
        case TN_INT64: return launch<int64_t, SUM, ARG, MIN>(src, axis, out, s);
        case TN_FLOAT16: return launch<__half, SUM, ARG, MIN>(src, axis, out, s);
        case TN_BFLOAT16: return launch<__nv_bfloat16, SUM, ARG, MIN>(src, axis, out, s);
        case TN_FLOAT32: return launch<float, SUM, ARG, MIN>(src, axis, out, s);
        case TN_FLOAT64: return launch<double, SUM, ARG, MIN>(src, axis, out, s);
        default: return fail(TN_UNSUPPORTED_DTYPE, "reduction: dtype %d unsupported", (int)src->dtype);
    }
}

tn_status check(const tn_tensor_t* src, const tn_tensor_t* dst, uint8_t axis, bool index_out, bool floats_only) {
    if (!src || !dst) return fail(TN_ERROR, "null tensor");
    if (axis >= src->rank) return fail(TN_ERROR, "axis %d out of range for rank %d", (int)axis, (int)src->rank);
    if (floats_only ? !is_float(src->dtype) : !is_numeric(src->dtype))
        return fail(TN_UNSUPPORTED_DTYPE, "reduction: dtype %d unsupported", (int)src->dtype);
    if (index_out ? dst->dtype != TN_INT64 : dst->dtype != src->dtype)
        return fail(TN_UNSUPPORTED_DTYPE, "reduction: result dtype %d does not fit source dtype %d", (int)dst->dtype,
                    (int)src->dtype);
    if (src->environment.kind != TN_DEVICE || dst->environment.kind != TN_DEVICE ||
        src->environment.resource.device.id != dst->environment.resource.device.id)
        return fail(TN_INCOMPATIBLE_DEVICES, "operands must live on one device");
    int64_t expect = 1;
    for (int d = 0; d < src->rank; ++d)
        if (d != axis) expect *= (int64_t)src->shape.sizes[d];
    if ((int64_t)dst->size != expect)
        return fail(TN_ERROR, "reduction: result holds %zu elements, expected %lld", dst->size, (long long)expect);
    return use_device_of(dst);
}

// ------------------------------------------------------------------ fixed scratch ------
// Scratch for tn_argsum_fixed_scratch: a region that is part of the loaded module instead of
// coming from an allocator. Every GPU that loads the library carries these 192 KiB until the
// process exits. Host code must not hand `g_fixed_scratch` itself to a kernel (on the host the
// name is only a handle for the symbol); its device address is looked up once per device below.
constexpr size_t kFixedScratchBytes = 192 * 1024;
constexpr int kMaxDevices = 64;
static __device__ __align__(256) unsigned char g_fixed_scratch[kFixedScratchBytes];

std::mutex g_fixed_mutex;
void* g_fixed_address[kMaxDevices] = {nullptr};

// Device address of the scratch region on `device`, which must be the current device.
tn_status fixed_scratch_address(int device, void** out) {
    if (device < 0 || device >= kMaxDevices) return fail(TN_ERROR, "device id %d is beyond the %d this entry point tracks", device, kMaxDevices);
    std::lock_guard<std::mutex> lock(g_fixed_mutex);
    if (g_fixed_address[device] == nullptr) {
        void* ptr = nullptr;
        cudaError_t err = cudaGetSymbolAddress(&ptr, g_fixed_scratch);
        if (err != cudaSuccess || ptr == nullptr) {
            cudaGetLastError();
            return fail(TN_ERROR, "cudaGetSymbolAddress(fixed scratch) failed on device %d: %s", device, cudaGetErrorString(err));
        }
        g_fixed_address[device] = ptr;
    }
    *out = g_fixed_address[device];
    return TN_SUCCESS;
}

template <typename T>
tn_status launch_sum_fixed(const T* p, int64_t rows, int64_t len, Outputs out, void* scratch, cudaStream_t s) {
    const size_t capacity = kFixedScratchBytes / sizeof(Partial<T>);
    if ((size_t)rows > capacity)
        return fail(TN_ERROR, "argsum_fixed_scratch: %lld rows need more than the %zu-byte fixed scratch region (at most %zu rows of this dtype)",
                    (long long)rows, kFixedScratchBytes, capacity);
    const int64_t row_bytes = len * (int64_t)sizeof(T);
    int64_t splits = ceil_div((int64_t)sm_count() * 4, rows);
    const int64_t by_length = ceil_div(row_bytes, int64_t(64) << 10);
    if (splits > by_length) splits = by_length;
    if (splits > (int64_t)(capacity / (size_t)rows)) splits = (int64_t)(capacity / (size_t)rows);
    if (splits > 1024) splits = 1024;
    if (splits < 1) splits = 1;
    Partial<T>* partials = static_cast<Partial<T>*>(scratch);
    // stage 1 writes every (row, segment) slot that stage 2 reads, so nothing left in the region
    // by an earlier call is ever consumed and no clearing pass is needed
    reduce_split_partial<T, true, false, false><<<dim3((unsigned)splits, (unsigned)rows), kThreads, 0, s>>>(p, len, (int)splits, partials);
    TN_TRY(after_launch("reduce_split_partial (fixed scratch)"));
    reduce_split_final<T, true, false, false><<<(unsigned)rows, 32, 0, s>>>(p, rows, len, (int)splits, partials, out);
    return after_launch("reduce_split_final (fixed scratch)");
}

}  // namespace

tn_status reduce_abort_count(unsigned int* count) {
    TN_CUDA(cudaMemcpyFromSymbol(count, g_reduce_aborts, sizeof(unsigned int)));
    return TN_SUCCESS;
}

}  // namespace tnb

using namespace tnb;

extern "C" {

tn_status tn_argmax(const tn_tensor_t* src, tn_tensor_t* dst, tn_stream_t stream, uint8_t axis) {
    TN_TRY(check(src, dst, axis, true, false));
    return by_dtype<false, true, false>(src, axis, Outputs{nullptr, nullptr, static_cast<int64_t*>(dst->address), 0}, as_cuda(stream));
}

tn_status tn_argmin(const tn_tensor_t* src, tn_tensor_t* dst, tn_stream_t stream, uint8_t axis) {
    TN_TRY(check(src, dst, axis, true, false));
    return by_dtype<false, true, true>(src, axis, Outputs{nullptr, nullptr, static_cast<int64_t*>(dst->address), 0}, as_cuda(stream));
}

tn_status tn_argsum(const tn_tensor_t* src, tn_tensor_t* dst, tn_stream_t stream, uint8_t axis) {
    TN_TRY(check(src, dst, axis, false, false));
    return by_dtype<true, false, false>(src, axis, Outputs{dst->address, nullptr, nullptr, 0}, as_cuda(stream));
}

tn_status tn_argmean(const tn_tensor_t* src, tn_tensor_t* dst, tn_stream_t stream, uint8_t axis) {
    TN_TRY(check(src, dst, axis, false, true));  // floats only, src/cpu/argred.cpp:304-315
    return by_dtype<true, false, false>(src, axis, Outputs{dst->address, nullptr, nullptr, 1}, as_cuda(stream));
}

tn_status tn_max(const tn_tensor_t* src, tn_tensor_t* dst, tn_stream_t stream, uint8_t axis) {
    TN_TRY(check(src, dst, axis, false, false));
    return by_dtype<false, true, false>(src, axis, Outputs{nullptr, dst->address, nullptr, 0}, as_cuda(stream));
}

tn_status tn_reduce_stats(const tn_tensor_t* src, tn_tensor_t* max_out, tn_tensor_t* sum_out, tn_tensor_t* argmax_out,
                          tn_stream_t stream, uint8_t axis) {
    if (!max_out && !sum_out && !argmax_out) return fail(TN_ERROR, "reduce_stats: no output requested");
    if (max_out) TN_TRY(check(src, max_out, axis, false, false));
    if (sum_out) TN_TRY(check(src, sum_out, axis, false, false));
    if (argmax_out) TN_TRY(check(src, argmax_out, axis, true, false));
    Outputs out{sum_out ? sum_out->address : nullptr, max_out ? max_out->address : nullptr,
                argmax_out ? static_cast<int64_t*>(argmax_out->address) : nullptr, 0};
    return by_dtype<true, true, false>(src, axis, out, as_cuda(stream));
}

// Sum along the LAST axis of a dense tensor with the two-kernel split reduction, taking its
// partial-sum workspace from a fixed region built into the library instead of from an allocator.
//
// Who needs this: hosts that are not allowed to allocate device memory at the point where they
// call in. Typical cases are a serving process that sized every device buffer at start-up and
// has nothing left for (or forbids) later driver or pool allocations, and callers on a path
// where the locking and implicit synchronisation of an allocation call are unacceptable.
// tn_argsum may take scratch from the stream-ordered pool; this entry point never calls
// cudaMalloc, cudaMallocAsync, cudaFree or any other allocating routine.
//
// Limits and rules:
//   - the workspace is 192 KiB per GPU, resident from library load to process exit;
//   - the source must be dense row-major and `axis` its last axis; the region holds one partial
//     result per (row, segment), so a call takes at most 192 KiB / sizeof(partial) rows: 8192 for
//     float32, float64 and the integer types (24-byte partials), 12288 for float16 and bfloat16
//     (16-byte partials); fewer segments per row are used as the row count grows. More rows are
//     refused with TN_ERROR and a message that names the limit;
//   - a zero-length last axis gives sums of zero, like tn_argsum (the result is cleared with a
//     memset on the stream; nothing is launched);
//   - the first call on each device looks the region's device address up
//     (cudaGetSymbolAddress, with that device current) and remembers it; make that first call
//     outside any stream capture;
//   - all calls on a device share the one region and it keeps whatever the previous call left
//     there. Each call overwrites every slot it later reads, so stale contents are harmless,
//     but two calls whose kernels overlap on the GPU (different streams, no ordering) race on
//     it: order them on one stream or with events.
tn_status tn_argsum_fixed_scratch(const tn_tensor_t* src, tn_tensor_t* dst, tn_stream_t stream, uint8_t axis) {
    TN_TRY(check(src, dst, axis, false, false));
    if (axis != src->rank - 1) return fail(TN_ERROR, "argsum_fixed_scratch: axis %d is not the last axis of a rank-%d tensor", (int)axis, (int)src->rank);
    const int64_t len = (int64_t)src->shape.sizes[axis];
    if (dst->size == 0) return TN_SUCCESS;
    if (len == 0) {
        // an empty sum is zero for every row; tn_argsum writes the same
        TN_TRY(use_device_of(dst));
        TN_CUDA(cudaMemsetAsync(dst->address, 0, dst->size * (size_t)dtype_bytes(dst->dtype), as_cuda(stream)));
        return TN_SUCCESS;
    }
    int64_t expect = 1;
    for (int d = src->rank - 1; d >= 0; --d) {
        const int64_t sz = (int64_t)src->shape.sizes[d];
        if (sz != 1 && src->strides.sizes[d] != expect) return fail(TN_ERROR, "argsum_fixed_scratch: the source must be dense row-major");
        expect *= sz;
    }
    const int64_t rows = expect / len;
    void* scratch = nullptr;
    TN_TRY(fixed_scratch_address(dst->environment.resource.device.id, &scratch));
    const Outputs out{dst->address, nullptr, nullptr, 0};
    cudaStream_t s = as_cuda(stream);
    switch (src->dtype) {
        case TN_INT8: return launch_sum_fixed(static_cast<const int8_t*>(src->address), rows, len, out, scratch, s);
        case TN_INT16: return launch_sum_fixed(static_cast<const int16_t*>(src->address), rows, len, out, scratch, s);
        case TN_INT32: return launch_sum_fixed(static_cast<const int32_t*>(src->address), rows, len, out, scratch, s);
        case TN_INT64: return launch_sum_fixed(static_cast<const int64_t*>(src->address), rows, len, out, scratch, s);
        case TN_FLOAT16: return launch_sum_fixed(static_cast<const __half*>(src->address), rows, len, out, scratch, s);
        case TN_BFLOAT16: return launch_sum_fixed(static_cast<const __nv_bfloat16*>(src->address), rows, len, out, scratch, s);
        case TN_FLOAT32: return launch_sum_fixed(static_cast<const float*>(src->address), rows, len, out, scratch, s);
        case TN_FLOAT64: return launch_sum_fixed(static_cast<const double*>(src->address), rows, len, out, scratch, s);
        default: return fail(TN_UNSUPPORTED_DTYPE, "argsum_fixed_scratch: dtype %d unsupported", (int)src->dtype);
    }
}

}  // extern "C"
