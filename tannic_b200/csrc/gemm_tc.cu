// Batched GEMM on the 5th-generation tensor cores of sm_100a: tcgen05.mma with the fp32
// accumulator in tensor memory, operands staged in shared memory by TMA through a multistage
// mbarrier pipeline, warp-specialised roles, persistent CTAs (one per SM).
//
//   warp 0      TMA producer   (one elected lane issues cp.async.bulk.tensor loads)
//   warp 1      MMA issuer     (one elected lane issues tcgen05.mma / tcgen05.commit)
//   warps 2..9  epilogue       (tcgen05.ld -> convert -> shared memory -> global: 32-row x 64-byte
//                               boxes handed to TMA where the result's base and pitches are
//                               multiples of 16 bytes, else coalesced element stores; each warp
//                               owns the TMEM lane quarter (warp % 4) and every second 32-column
//                               chunk, or every chunk when only four epilogue warps run)
//
// Three operand modes share the main loop:
//   MODE_K  B is K-major ([N, K]: `matmul(X, W.transpose(-1,-2))`), one 64x256 TMA box per stage;
//   MODE_N  B is N-major ([K, N]: plain matmul, the [Cin, H*W] matrix of a 1x1 convolution),
//           four 64-column boxes per stage and MN-major shared-memory descriptors;
//           (with K <= 256 and one A for all batches: the stationary-A kernel further down);
//   MODE_CONV  implicit-GEMM convolution: A = weights repacked to [tap][Cout][Cin], B = the
//           activation in NHWC, fetched per (tap, channel block) as a 4-D box
//           {64 channels, Wout, Hbox, 1} whose W/H coordinates are shifted by the tap and may
//           run out of range (TMA zero fill = zero padding). A tile is Hbox full output rows,
//           so the accumulator [Cout tile, Hbox*Wout pixels] stores straight into NCHW.
//
// CTA tile 128 x 256 x 64: one UMMA is M=128, N=256, K=16, so a K-block is four MMAs. The
// 512 TMEM columns hold two 128x256 fp32 accumulators, so the epilogue of tile i overlaps the
// main loop of tile i+1. No multicast is used anywhere: every CTA issues its own TMA loads and
// L2 provides the reuse between neighbouring tiles.
//
// Every wait on an mbarrier is bounded. When a wait runs out the CTA raises an abort flag, all
// roles leave their loops, outstanding TMA transactions are given time to land, tensor memory
// is released and a device-side error counter is incremented (read by tn_device_errors()).
#include "gemm_tc.cuh"

#include <cuda.h>

#include <cstdlib>
#include <mutex>

namespace tnb {
namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;            // 64 x 2 bytes = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int PACKED_STAGES = 2;                 // operand stages of the packed-epilogue variant
constexpr int kEpilogueWarps = 8;                // two per TMEM lane quarter, interleaved over 32-column chunks
constexpr int kThreads = 64 + 32 * kEpilogueWarps;
constexpr uint32_t A_BYTES = BM * BK * 2;        // 16 KiB
constexpr uint32_t B_BYTES = BN * BK * 2;        // 32 KiB
constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
constexpr uint32_t TMEM_COLS = 512;              // two accumulators of BN fp32 columns
constexpr int STAGING_PITCH = 17;                // words per staged row of the element-wise path (conflict-free transpose)
constexpr uint32_t STAGING_WARP_BYTES = 4096;    // per epilogue warp: two 2 KiB boxes for TMA stores (or one 32 x 80 B block)
constexpr uint32_t STAGING_BYTES = kEpilogueWarps * STAGING_WARP_BYTES;
constexpr uint32_t SMEM_BYTES = 1024 /*alignment slack*/ + STAGES * STAGE_BYTES + STAGING_BYTES + 256 /*barriers*/;
// packed epilogue: a warp stages 32 rows of up to BN 16-bit columns plus the offset from a 16-byte boundary
constexpr uint32_t PACK_STAGE_MAX = (32 * BN * 2 + 16 + 127) & ~127u;
constexpr uint32_t PACKED_SMEM_MAX = 1024 + PACKED_STAGES * STAGE_BYTES + kEpilogueWarps * PACK_STAGE_MAX + 256;
static_assert(PACKED_SMEM_MAX <= 232448, "packed epilogue exceeds the shared memory of an SM");

constexpr uint32_t kSpinFast = 2048;      // polls without sleeping
constexpr uint32_t kSpinLimit = 1u << 20; // then ~64 ns sleeps: gives up after roughly 0.1 s

__device__ unsigned int g_tc_aborts = 0;
std::atomic<uint64_t> g_path_launches[4];  // general, packed rows, packed rows + statistics, stationary A

// ------------------------------------------------------------------ PTX wrappers ------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}
// Bounded wait. Returns false when the CTA is aborting (this wait or another one ran out).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, uint32_t limit = kSpinLimit) {
    for (uint32_t it = 0; it < limit; ++it) {
        if (mbar_test(bar, parity)) return true;
        if (it >= kSpinFast) {
            if (*abort_flag) return false;
            __nanosleep(64);
        }
    }
    *abort_flag = 1;
    return false;
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

// Result tiles leave through TMA as well: a warp writes a 32-row x 64-byte box into shared memory
// (64-byte swizzle) and one lane hands it to the copy engine, which clips it at the tensor's edges.
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
        ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
// Untiled copy of a 16-byte-aligned shared-memory range to a 16-byte-aligned global range.
__device__ __forceinline__ void bulk_store_linear(void* dst, uint32_t src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
        ::"l"(reinterpret_cast<uint64_t>(dst)), "r"(src), "r"(bytes)
        : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// until at most one of this thread's store groups still reads its shared-memory source
__device__ __forceinline__ void bulk_wait_read_1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// tcgen05.ld is asynchronous: the registers are valid only after tcgen05.wait::ld. The wait
// below names the registers as read-write operands so that no use of them can be scheduled
// ahead of it.
__device__ __forceinline__ void tmem_load_issue(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32"
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15,"
        " %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_load_wait(uint32_t (&v)[32]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
        : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]),
          "+r"(v[8]), "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15]),
          "+r"(v[16]), "+r"(v[17]), "+r"(v[18]), "+r"(v[19]), "+r"(v[20]), "+r"(v[21]), "+r"(v[22]), "+r"(v[23]),
          "+r"(v[24]), "+r"(v[25]), "+r"(v[26]), "+r"(v[27]), "+r"(v[28]), "+r"(v[29]), "+r"(v[30]), "+r"(v[31])
        :
        : "memory");
}

// Registers -> tensor memory, the mirror image of the load above: lane i of the warp writes 32
// consecutive 32-bit columns of TMEM lane (32 * (warp % 4) + i).
__device__ __forceinline__ void tmem_store(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0],"
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16,"
        " %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
          "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
          "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
          "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
}
__device__ __forceinline__ void tmem_store_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// The same MMA with the A operand in tensor memory: row i of the 128 x 16 block in lane i, two
// consecutive K elements per 32-bit column (so one instruction reads 8 columns).
__device__ __forceinline__ void umma_f16_a_tmem(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Shared-memory matrix descriptor of a 128-byte-swizzled tile (sm_100 format: start address,
// leading / stride byte offsets in 16-byte units, version 1 at bit 46, layout type 2 =
// SWIZZLE_128B at bits 61-63).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((addr & 0x3FFFF) >> 4);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

enum { MODE_K = 0, MODE_N = 1, MODE_CONV = 2 };

struct KernelArgs {
    void* d;
    const void* bias;
    int64_t M, N;              // result rows / columns per batch (conv: Cout, Hout*Wout)
    int64_t ldd, d_batch;
    int m_tiles, n_tiles;
    uint32_t total_tiles;
    int k_blocks;              // 64-wide K blocks per tile (conv: taps * channel blocks)
    int tile_n;                // result columns per tile (256; conv: Hbox * Wout)
    int umma_n;                // N of the MMA instruction (multiple of 16, >= tile_n)
    uint32_t stage_tx;         // bytes TMA delivers per stage
    int a_batched, b_batched;  // 0: operand shared by all batches (batch coordinate pinned to 0)
    int is_bf16;               // operand format: 1 = bf16, 0 = fp16
    int d_is_f32;
    int vec_store;             // result rows can be written with 16-byte stores
    int tma_store;             // result leaves through TMA boxes (map_d is valid)
    int has_scale;
    float scale;
    // convolution geometry
    int cblocks, kw, pad_h, pad_w, hbox, str_h;
    int epi_warps;             // 4 or 8 epilogue warps take part (the others exit at once)
    uint32_t pack_stage_bytes; // packed epilogue: bytes of one warp's staging block (multiple of 128)
    // mirrored results: the same tile is also written, at the same offsets, into these buffers (other GPUs' memory
    // mapped into this process); 16-bit results through the 16-byte store path only
    void* mirror[7];
    int n_mirrors;
    // stationary-A variant
    const void* a;             // first operand [M, K], K contiguous
    int64_t lda;
    int k_total;               // K (a multiple of 8, at most 256)
    int groups;                // CTA groups; each holds every row tile once and takes a share of the column tiles
    uint32_t col_tiles;        // column tiles over all batches
    void* stat_max;            // fused row statistics (packed epilogue only); each may be null
    void* stat_sum;
    int64_t* stat_argmax;
};

// Tiles are walked in groups of 16 row-tiles so that the CTAs running at the same time share
// rows of A and columns of B in L2.
constexpr int kGroupM = 16;
__device__ __forceinline__ void tile_coords(uint32_t t, int m_tiles, int n_tiles, int& batch, int& mt, int& nt) {
    // tile counts are below 2^31 (checked on the host): 32-bit divisions only
    const uint32_t per_batch = static_cast<uint32_t>(m_tiles) * static_cast<uint32_t>(n_tiles);
    batch = static_cast<int>(t / per_batch);
    int r = static_cast<int>(t - static_cast<uint32_t>(batch) * per_batch);
    const int group_span = kGroupM * n_tiles;
    const int g = r / group_span;
    r -= g * group_span;
    const int rows_in_group = min(kGroupM, m_tiles - g * kGroupM);
    nt = r / rows_in_group;
    mt = g * kGroupM + (r - nt * rows_in_group);
}

// Accumulator -> result element: bias, rounding to the result type, optional scalar factor
// (applied to the rounded value and rounded again, like `matmul(...) * scalar` in two kernels).
template <typename OutT, bool SCALE>
__device__ __forceinline__ OutT finish(float acc, float scale, float bias) {
    const float v = acc + bias;
    if constexpr (std::is_same<OutT, float>::value) {
        return SCALE ? v * scale : v;
    } else {
        OutT r = from_compute<OutT, float>(v);
        if constexpr (SCALE) r = from_compute<OutT, float>(to_compute<float>(r) * scale);
        return r;
    }
}

// Two accumulators -> a packed pair of result elements: one conversion instruction for both,
// and the optional scalar factor as one packed multiply. The product of two 16-bit floats is
// exact in fp32, so the packed multiply rounds exactly like `float(a) * float(s)` rounded once.
template <typename OutT> __device__ __forceinline__ uint32_t pair_of(float s);
template <> __device__ __forceinline__ uint32_t pair_of<__half>(float s) {
    const __half2 h = __float2half2_rn(s);
    return *reinterpret_cast<const uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pair_of<__nv_bfloat16>(float s) {
    const __nv_bfloat162 h = __float2bfloat162_rn(s);
    return *reinterpret_cast<const uint32_t*>(&h);
}
template <typename OutT, bool SCALE> __device__ __forceinline__ uint32_t finish_pair(float lo, float hi, uint32_t scale2);
template <> __device__ __forceinline__ uint32_t finish_pair<__half, false>(float lo, float hi, uint32_t) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t finish_pair<__half, true>(float lo, float hi, uint32_t scale2) {
    const __half2 h = __hmul2(__floats2half2_rn(lo, hi), *reinterpret_cast<const __half2*>(&scale2));
    return *reinterpret_cast<const uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t finish_pair<__nv_bfloat16, false>(float lo, float hi, uint32_t) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t finish_pair<__nv_bfloat16, true>(float lo, float hi, uint32_t scale2) {
    const __nv_bfloat162 h = __hmul2(__floats2bfloat162_rn(lo, hi), *reinterpret_cast<const __nv_bfloat162*>(&scale2));
    return *reinterpret_cast<const uint32_t*>(&h);
}

struct EpilogueTile {
    uint8_t* dbase;      // result of this batch
    int64_t ldd;
    int64_t row0;        // first result row of this warp
    int rows;            // valid rows (<= 32)
    int64_t col_base;    // first result column of the tile
    int64_t col_end;     // one past the last column this tile owns
    uint32_t taddr0;     // TMEM address of (lane quarter, accumulator buffer)
    int chunk0;          // first 32-column chunk of this warp
    int chunk_step;      // 1: this warp takes every chunk, 2: every second one
    float bias, scale;
    int vec_store;
    int has_bias;
    int tma_store;
    int batch;
    int64_t n_total;     // columns of the whole result
    const CUtensorMap* map_d;
    void* const* mirrors;  // n_mirrors further result buffers of the same layout (peer memory), or null
    int n_mirrors;
    int64_t batch_elems;   // element offset of this batch inside a result buffer
};

// Writes one 32 x 32 block (lane = row, v = 32 consecutive columns starting at col0) through a
// per-warp staging area so that the global stores run along rows. OutT and SCALE are
// compile-time so that the per-element conversion code has no branches.
template <typename OutT, bool SCALE>
__device__ __forceinline__ void store_block(const EpilogueTile& e, uint32_t (&v)[32], int64_t col0, uint8_t* stage, int lane, int& flip) {
    uint32_t* stage_words = reinterpret_cast<uint32_t*>(stage);
    if (e.has_bias) {  // warp-uniform
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) + e.bias);
    }
    // A box may run past the edge of the result (TMA clips it) but not into columns that belong
    // to the next tile, which happens only where a convolution tile is not a multiple of 32 wide.
    if (e.tma_store && (col0 + 32 <= e.col_end || e.col_end == e.n_total)) {  // warp-uniform
        constexpr bool kF32 = std::is_same<OutT, float>::value;
        const int x = (lane >> 1) & 3;  // 64-byte swizzle: 16-byte unit q of row r sits in unit q ^ ((r >> 1) & 3)
#pragma unroll
        for (int h = 0; h < (kF32 ? 2 : 1); ++h) {
            uint8_t* buf = stage + (flip & 1) * 2048;
            flip ^= 1;
            if (lane == 0) bulk_wait_read_1();  // the store that used this buffer two boxes ago has read it
            __syncwarp();
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                uint32_t w[4];
                if constexpr (kF32) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) w[j] = __float_as_uint(finish<float, SCALE>(__uint_as_float(v[h * 16 + 4 * q + j]), e.scale, 0.0f));
                } else {
                    const uint32_t scale2 = pair_of<OutT>(e.scale);
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        w[j] = finish_pair<OutT, SCALE>(__uint_as_float(v[8 * q + 2 * j]), __uint_as_float(v[8 * q + 2 * j + 1]), scale2);
                }
                *reinterpret_cast<uint4*>(buf + lane * 64 + ((q ^ x) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
            }
            fence_async_smem();  // generic-proxy writes become visible to the copy engine
            __syncwarp();
            if (lane == 0) {
                tma_store_3d(e.map_d, smem_u32(buf), static_cast<int>(col0) + h * 16, static_cast<int>(e.row0), e.batch);
                bulk_commit();
            }
        }
        return;
    }
    if (e.tma_store) {
        if (lane == 0) bulk_wait_read_0();  // the element-wise path below reuses the boxes' memory
    }
    __syncwarp();  // the previous block's readers are done with the staging area
    if constexpr (!std::is_same<OutT, float>::value) {
        // rows of 64 bytes at an 80-byte pitch: conflict-free both for the 16-byte writes of a
        // lane's own row and for reads along a row
        const uint32_t scale2 = pair_of<OutT>(e.scale);
        uint4* mine = reinterpret_cast<uint4*>(stage + lane * 80);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
                w[j] = finish_pair<OutT, SCALE>(__uint_as_float(v[8 * q + 2 * j]), __uint_as_float(v[8 * q + 2 * j + 1]), scale2);
            mine[q] = make_uint4(w[0], w[1], w[2], w[3]);
        }
        __syncwarp();
        if (e.vec_store) {
            // 8 rows x 4 lanes x 16 bytes per store instruction
            const int seg = lane & 3;
            const int64_t col = col0 + seg * 8;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int r = i * 8 + (lane >> 2);
                if (r < e.rows && col < e.col_end) {
                    const uint4 val = *reinterpret_cast<const uint4*>(stage + r * 80 + seg * 16);
                    const int64_t at = (e.row0 + r) * e.ldd + col;
                    *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(e.dbase) + at) = val;
                    // the same 16 bytes into every mirror (plain stores into peer memory: NVLink carries them while
                    // the tensor cores work on the next tile)
                    for (int m = 0; m < e.n_mirrors; ++m)
                        *reinterpret_cast<uint4*>(static_cast<uint16_t*>(e.mirrors[m]) + e.batch_elems + at) = val;
                }
            }
        } else {
            // any alignment: one row of 32 elements per store instruction
            const int64_t col = col0 + lane;
            if (col < e.col_end) {
                uint16_t* out = reinterpret_cast<uint16_t*>(e.dbase) + e.row0 * e.ldd + col;
                const uint16_t* src = reinterpret_cast<const uint16_t*>(stage) + lane;
                if (e.rows == 32) {
#pragma unroll
                    for (int r = 0; r < 32; ++r) out[r * e.ldd] = src[r * 40];
                } else {
                    for (int r = 0; r < e.rows; ++r) out[r * e.ldd] = src[r * 40];
                }
            }
        }
    } else {
        // fp32 result: two passes of 16 columns through the same staging area
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            if (h) __syncwarp();
            const int64_t colh = col0 + h * 16;
            if (e.vec_store) {
                uint4* mine = reinterpret_cast<uint4*>(stage + lane * 80);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    uint32_t w[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) w[j] = __float_as_uint(finish<float, SCALE>(__uint_as_float(v[h * 16 + 4 * q + j]), e.scale, 0.0f));
                    mine[q] = make_uint4(w[0], w[1], w[2], w[3]);
                }
                __syncwarp();
                const int seg = lane & 3;
                const int64_t col = colh + seg * 4;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int r = i * 8 + (lane >> 2);
                    if (r < e.rows && col < e.col_end)
                        *reinterpret_cast<uint4*>(reinterpret_cast<float*>(e.dbase) + (e.row0 + r) * e.ldd + col) =
                            *reinterpret_cast<const uint4*>(stage + r * 80 + seg * 16);
                }
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    stage_words[lane * STAGING_PITCH + j] = __float_as_uint(finish<float, SCALE>(__uint_as_float(v[h * 16 + j]), e.scale, 0.0f));
                __syncwarp();
                const int64_t col = colh + (lane & 15);
                if (col < e.col_end) {
                    float* out = reinterpret_cast<float*>(e.dbase) + e.row0 * e.ldd + col;
                    for (int r = lane >> 4; r < e.rows; r += 2) out[r * e.ldd] = __uint_as_float(stage_words[r * STAGING_PITCH + (lane & 15)]);
                }
            }
        }
    }
}

// Drains this warp's share of the accumulator: 32 rows, every second 32-column chunk. The
// TMEM load of the next chunk is in flight while the current one is converted and stored.
template <typename OutT, bool SCALE>
__device__ __forceinline__ void drain_tile(const EpilogueTile& e, uint8_t* stage, int lane, int& flip) {
    if (e.rows <= 0) return;  // warp-uniform
    auto valid = [&](int c) { return c < BN / 32 && e.col_base + c * 32 < e.col_end; };
    uint32_t va[32], vb[32];
    int c = e.chunk0;
    if (!valid(c)) return;
    tmem_load_issue(e.taddr0 + c * 32, va);
    while (true) {
        tmem_load_wait(va);
        const int c2 = c + e.chunk_step;
        const bool more2 = valid(c2);
        if (more2) tmem_load_issue(e.taddr0 + c2 * 32, vb);
        store_block<OutT, SCALE>(e, va, e.col_base + c * 32, stage, lane, flip);
        if (!more2) break;
        tmem_load_wait(vb);
        c = c2 + e.chunk_step;
        const bool more = valid(c);
        if (more) tmem_load_issue(e.taddr0 + c * 32, va);
        store_block<OutT, SCALE>(e, vb, e.col_base + c2 * 32, stage, lane, flip);
        if (!more) break;
    }
}

// ---- packed epilogue -------------------------------------------------------------------
// A result whose rows are NOT a multiple of 16 bytes (197 bfloat16 columns, say) defeats both the
// TMA boxes and 16-byte row stores. But when the rows follow one another without a gap (pitch ==
// columns) and one tile spans all columns, the 32 rows a warp drains are ONE contiguous byte range
// of global memory. The warp builds that range in shared memory exactly as it will lie in global
// memory, at the same offset from a 16-byte boundary, and hands its 16-byte-aligned middle to the
// copy engine as a single untiled bulk store; the up to seven elements before and after the
// aligned part are written with 2-byte stores. One warp drains all column chunks of its 32 rows,
// so nothing is shared between warps: warps 2-5 take the tiles in accumulator 0, warps 6-9 those
// in accumulator 1.

// Both halves of a packed pair as float32.
template <typename OutT> __device__ __forceinline__ void unpack_pair(uint32_t w, float& lo, float& hi);
template <> __device__ __forceinline__ void unpack_pair<__nv_bfloat16>(uint32_t w, float& lo, float& hi) {
    lo = __uint_as_float(w << 16);
    hi = __uint_as_float(w & 0xFFFF0000u);
}
template <> __device__ __forceinline__ void unpack_pair<__half>(uint32_t w, float& lo, float& hi) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
    lo = f.x;
    hi = f.y;
}
template <typename OutT> __device__ __forceinline__ uint32_t max_pair(uint32_t a, uint32_t b);
template <> __device__ __forceinline__ uint32_t max_pair<__nv_bfloat16>(uint32_t a, uint32_t b) {
    const __nv_bfloat162 m = __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
    return *reinterpret_cast<const uint32_t*>(&m);
}
template <> __device__ __forceinline__ uint32_t max_pair<__half>(uint32_t a, uint32_t b) {
    const __half2 m = __hmax2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
    return *reinterpret_cast<const uint32_t*>(&m);
}

// Row statistics of the rounded results, kept by the lane that drains the row: the sum in float32,
// and for the maximum of the even and of the odd columns its value and the 32-column chunk in which
// it first appeared (a strict, ordered comparison: a NaN is never selected, the first of equal
// values stays). The column itself is looked up once, after the last chunk.
struct RowStats {
    float sum0, sum1;
    float max_even, max_odd;
    int chunk_even, chunk_odd;
    __device__ __forceinline__ void init() {
        sum0 = sum1 = 0.0f;
        max_even = max_odd = -INFINITY;
        chunk_even = chunk_odd = -1;
    }
    template <typename OutT>
    __device__ __forceinline__ void update(const uint32_t (&w)[16], int ncols, int chunk) {
        float lo, hi;
        float best_even = -INFINITY, best_odd = -INFINITY;
        if (ncols == 32) {  // warp-uniform
            uint32_t m[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) m[j] = max_pair<OutT>(w[j], w[j + 8]);
#pragma unroll
            for (int j = 0; j < 4; ++j) m[j] = max_pair<OutT>(m[j], m[j + 4]);
            m[0] = max_pair<OutT>(max_pair<OutT>(m[0], m[2]), max_pair<OutT>(m[1], m[3]));
            unpack_pair<OutT>(m[0], best_even, best_odd);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                unpack_pair<OutT>(w[j], lo, hi);
                sum0 += lo;
                sum1 += hi;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                unpack_pair<OutT>(w[j], lo, hi);
                if (2 * j < ncols) {
                    sum0 += lo;
                    best_even = fmaxf(best_even, lo);
                }
                if (2 * j + 1 < ncols) {
                    sum1 += hi;
                    best_odd = fmaxf(best_odd, hi);
                }
            }
        }
        if (best_even > max_even) {
            max_even = best_even;
            chunk_even = chunk;
        }
        if (best_odd > max_odd) {
            max_odd = best_odd;
            chunk_odd = chunk;
        }
    }
};

// Stages 32 consecutive columns of this lane's row at `dst` (2-byte aligned). Full chunks are
// written as aligned 32-bit words: a lane whose row starts on an odd element shifts its packed
// pairs by one element (funnel shift) and writes the first and last element on their own.
// Accumulators of 32 consecutive columns -> 16 packed pairs of rounded (and scaled) results.
template <typename OutT, bool SCALE>
__device__ __forceinline__ void pack_chunk(const uint32_t (&v)[32], uint32_t (&w)[16], bool has_bias, float bias, uint32_t scale2) {
    if (has_bias) {  // warp-uniform
#pragma unroll
        for (int j = 0; j < 16; ++j)
            w[j] = finish_pair<OutT, SCALE>(__uint_as_float(v[2 * j]) + bias, __uint_as_float(v[2 * j + 1]) + bias, scale2);
    } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) w[j] = finish_pair<OutT, SCALE>(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]), scale2);
    }
}

// Stages the 16 pairs at `dst` (2-byte aligned). Full chunks are written as aligned 32-bit words: a
// lane whose row starts on an odd element shifts its packed pairs by one element (funnel shift) and
// writes the first and last element on their own.
__device__ __forceinline__ void stage_packed_chunk(const uint32_t (&w)[16], uint8_t* dst, int ncols) {
    if (ncols == 32) {  // warp-uniform
        const uint32_t odd = (static_cast<uint32_t>(reinterpret_cast<uintptr_t>(dst)) >> 1) & 1u;
        uint32_t* words = reinterpret_cast<uint32_t*>(dst + 2 * odd);
        const uint32_t shift = odd << 4;
#pragma unroll
        for (int j = 0; j < 15; ++j) words[j] = __funnelshift_r(w[j], w[j + 1], shift);
        if (odd) {
            *reinterpret_cast<uint16_t*>(dst) = static_cast<uint16_t>(w[0] & 0xFFFFu);
            *reinterpret_cast<uint16_t*>(dst + 62) = static_cast<uint16_t>(w[15] >> 16);
        } else {
            words[15] = w[15];
        }
    } else {
        uint16_t* out = reinterpret_cast<uint16_t*>(dst);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            if (2 * j < ncols) out[2 * j] = static_cast<uint16_t>(w[j] & 0xFFFFu);
            if (2 * j + 1 < ncols) out[2 * j + 1] = static_cast<uint16_t>(w[j] >> 16);
        }
    }
}

// Where the row statistics of a fused call go (any pointer may be null); `row` indexes all rows of
// all batches.
struct StatsOut {
    void* max;
    void* sum;
    int64_t* argmax;
};

// Drains rows [row0, row0 + rows) x all n columns of one accumulator into `stage` and sends them
// to the contiguous global range that starts at `gptr`.
template <typename OutT, bool SCALE, bool STATS>
__device__ __forceinline__ void drain_packed(uint8_t* stage, uint8_t* gptr, int n, int rows, uint32_t taddr0, bool has_bias, float bias, float scale,
                                             int lane, const StatsOut& so, int64_t first_row) {
    const uint32_t phase = static_cast<uint32_t>(reinterpret_cast<uintptr_t>(gptr)) & 15u;
    const int chunks = (n + 31) >> 5;
    const uint32_t scale2 = pair_of<OutT>(scale);
    uint8_t* my_row = stage + phase + static_cast<size_t>(lane) * n * 2;
    const bool mine = lane < rows;
    RowStats stats;
    stats.init();
    // One loop body for every chunk (the epilogue warps share the instruction cache with the producer
    // and the MMA issuer, so the code is kept small): the accumulators are packed into 16 registers,
    // then the load of the next chunk is issued into the freed ones and runs under the statistics
    // and the staging stores of this chunk.
    uint32_t v[32], w[16];
    tmem_load_issue(taddr0, v);
#pragma unroll 1
    for (int c = 0; c < chunks; ++c) {
        tmem_load_wait(v);
        pack_chunk<OutT, SCALE>(v, w, has_bias, bias, scale2);
        if (c + 1 < chunks) tmem_load_issue(taddr0 + (c + 1) * 32, v);
        const int ncols = min(32, n - c * 32);
        if (mine) {
            if constexpr (STATS) stats.template update<OutT>(w, ncols, c);
            stage_packed_chunk(w, my_row + c * 64, ncols);
        }
    }
    if constexpr (STATS) {
        if (mine) {
            // the chunk that holds the first occurrence of the row maximum: the even and the odd columns
            // each know theirs; equal maxima resolve to the earlier chunk, the scan below to the column
            int chunk = -1;
            float best = -INFINITY;
            if (stats.chunk_even >= 0) {
                chunk = stats.chunk_even;
                best = stats.max_even;
            }
            if (stats.chunk_odd >= 0 && (chunk < 0 || stats.max_odd > best || (stats.max_odd == best && stats.chunk_odd < chunk))) {
                chunk = stats.chunk_odd;
                best = stats.max_odd;
            }
            int index = 0;
            const OutT* row = reinterpret_cast<const OutT*>(my_row);
            if (chunk >= 0) {
                const int base = chunk * 32, width = min(32, n - base);
                index = base;
#pragma unroll 8
                for (int j = 31; j >= 0; --j)
                    if (j < width && to_compute<float>(row[base + j]) == best) index = base + j;
            }
            const int64_t r = first_row + lane;
            if (so.max) static_cast<OutT*>(so.max)[r] = row[index];  // the element itself: the sign of a zero survives
            if (so.sum) static_cast<OutT*>(so.sum)[r] = from_compute<OutT, float>(stats.sum0 + stats.sum1);
            if (so.argmax) so.argmax[r] = index;
        }
    }
    fence_async_smem();  // generic-proxy writes become visible to the copy engine
    __syncwarp();
    const uintptr_t g0 = reinterpret_cast<uintptr_t>(gptr), g1 = g0 + static_cast<size_t>(rows) * n * 2;
    const uintptr_t a0 = (g0 + 15) & ~uintptr_t(15), a1 = g1 & ~uintptr_t(15);
    const uintptr_t origin = g0 - phase;  // global address that corresponds to stage[0]
    if (lane == 0 && a1 > a0) {
        bulk_store_linear(reinterpret_cast<void*>(a0), smem_u32(stage + (a0 - origin)), static_cast<uint32_t>(a1 - a0));
        bulk_commit();
    }
    // elements before the first and after the last 16-byte boundary (at most seven each)
    const uintptr_t head_end = a0 < g1 ? a0 : g1;
    const uintptr_t tail_begin = a1 > a0 ? a1 : a0;
    if (lane < 8) {
        const uintptr_t x = g0 + 2 * lane;
        if (x < head_end) *reinterpret_cast<uint16_t*>(x) = *reinterpret_cast<const uint16_t*>(stage + (x - origin));
    } else if (lane < 16) {
        const uintptr_t x = tail_begin + 2 * (lane - 8);
        if (x < g1) *reinterpret_cast<uint16_t*>(x) = *reinterpret_cast<const uint16_t*>(stage + (x - origin));
    }
}

enum { OUT_F16 = 0, OUT_BF16 = 1, OUT_F32 = 2 };
template <int OUT> struct out_type { using type = __half; };
template <> struct out_type<OUT_BF16> { using type = __nv_bfloat16; };
template <> struct out_type<OUT_F32> { using type = float; };

// MODE: operand layout (see the top of the file); OUT: result element type; SCALE: multiply the
// rounded result by a scalar. All three are compile-time so that the epilogue is branch-free.
// PACK: PACK_ROWS selects the packed epilogue above (16-bit results only); it trades two of the
// four operand stages for 8 staging blocks of up to 16.5 KiB. PACK_STATS also produces the maximum,
// sum and argmax of every result row in the same pass.
enum { PACK_NONE = 0, PACK_ROWS = 1, PACK_STATS = 2 };
template <int MODE, int OUT, bool SCALE, int PACK>
__global__ void __launch_bounds__(kThreads, 1)
tc_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_d, const KernelArgs g) {
    constexpr bool PACKED = PACK != PACK_NONE;
    constexpr int kStages = PACKED ? PACKED_STAGES : STAGES;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;  // swizzled tiles need 1024-byte alignment
    uint8_t* base_ptr = smem_raw + (base - raw);
    const uint32_t staging_bytes = PACKED ? kEpilogueWarps * g.pack_stage_bytes : STAGING_BYTES;
    const uint32_t staging = base + kStages * STAGE_BYTES;
    uint8_t* staging_ptr = base_ptr + kStages * STAGE_BYTES;
    const uint32_t bars = staging + staging_bytes;
    // barrier layout (8 bytes each): full[kStages], empty[kStages], acc_full[2], acc_empty[2]
    const uint32_t full0 = bars, empty0 = bars + 8 * kStages, accf0 = bars + 16 * kStages, acce0 = accf0 + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + kStages * STAGE_BYTES + staging_bytes + 16 * kStages + 32);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_blocks = g.k_blocks;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(accf0 + 8 * b, 1);
            mbar_init(acce0 + 8 * b, PACKED ? 4 : g.epi_warps);  // packed: four warps per accumulator
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 2) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer ----
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (uint32_t t = blockIdx.x; ok && t < g.total_tiles; t += gridDim.x) {
                int batch, mt, nt;
                tile_coords(t, g.m_tiles, g.n_tiles, batch, mt, nt);
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % kStages;
                    const uint32_t parity = ((it / kStages) & 1) ^ 1;
                    if (!mbar_wait(empty0 + 8 * s, parity, abort_flag)) { ok = false; break; }
                    const uint32_t sa = base + s * STAGE_BYTES, sb = sa + A_BYTES;
                    mbar_expect_tx(full0 + 8 * s, g.stage_tx);
                    if constexpr (MODE == MODE_CONV) {
                        const int tap = kb / g.cblocks, cb = kb - tap * g.cblocks;
                        const int kh = tap / g.kw, kwi = tap - kh * g.kw;
                        tma_load_3d(sa, &map_a, full0 + 8 * s, cb * BK, mt * BM, tap);
                        // innermost coordinate (channels) is a multiple of 64; the W and H coordinates
                        // carry the tap shift and may be negative or past the edge (zero fill)
                        tma_load_4d(sb, &map_b, full0 + 8 * s, cb * BK, kwi - g.pad_w, nt * g.hbox * g.str_h + kh - g.pad_h, batch);
                    } else {
                        tma_load_3d(sa, &map_a, full0 + 8 * s, kb * BK, mt * BM, g.a_batched ? batch : 0);
                        if constexpr (MODE == MODE_N) {
                            // four boxes of 64 columns x BK rows, 8 KiB each
#pragma unroll
                            for (int c = 0; c < BN / 64; ++c)
                                tma_load_3d(sb + c * (64 * BK * 2), &map_b, full0 + 8 * s, nt * BN + c * 64, kb * BK, g.b_batched ? batch : 0);
                        } else {
                            tma_load_3d(sb, &map_b, full0 + 8 * s, kb * BK, nt * BN, g.b_batched ? batch : 0);
                        }
                    }
                }
            }
            if (!ok) {
                // give transactions that were already issued time to land before smem goes away
                for (int spin = 0; spin < 4096; ++spin) __nanosleep(64);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer ------
        if (lane == 0) {
            // instruction descriptor: D = F32 (bits 4-5 = 1), A/B format (bits 7-9, 10-12:
            // 0 = F16, 1 = BF16), B major (bit 16), N >> 3 (bits 17-22), M >> 4 (bits 24-28)
            const uint32_t fmt = g.is_bf16 ? 1u : 0u;
            const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((MODE == MODE_N ? 1u : 0u) << 16) |
                                   (static_cast<uint32_t>(g.umma_n >> 3) << 17) | (static_cast<uint32_t>(BM >> 4) << 24);
            uint32_t it = 0, local_tile = 0;
            bool ok = true;
            for (uint32_t t = blockIdx.x; ok && t < g.total_tiles; t += gridDim.x, ++local_tile) {
                const int buf = local_tile & 1;
                const uint32_t acc_parity = ((local_tile >> 1) & 1) ^ 1;
                if (!mbar_wait(acce0 + 8 * buf, acc_parity, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t tmem_acc = tmem_base + buf * BN;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % kStages;
                    const uint32_t parity = (it / kStages) & 1;
                    if (!mbar_wait(full0 + 8 * s, parity, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = base + s * STAGE_BYTES, sb = sa + A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // K-major: 16 elements = 32 bytes further along the swizzled row.
                        const uint64_t da = smem_desc(sa + k * UMMA_K * 2, 16, 1024);
                        // N-major: 16 k-rows of 128 bytes further; 64-column boxes are 8 KiB apart.
                        const uint64_t db = MODE == MODE_N ? smem_desc(sb + k * UMMA_K * 128, 64 * BK * 2, 1024)
                                                           : smem_desc(sb + k * UMMA_K * 2, 16, 1024);
                        umma_f16(tmem_acc, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(empty0 + 8 * s);  // frees the stage once these MMAs have read it
                }
                if (ok) umma_commit(accf0 + 8 * buf);  // accumulator complete
            }
        }
    } else if (PACKED) {
        // ------------------------------------------------------------ packed epilogue -
        if constexpr (PACKED) {
            const int ew = warp - 2;
            const int quarter = warp & 3;            // TMEM lanes [32*quarter, 32*quarter+32)
            const int buf = ew >> 2;                 // this warp drains the tiles of one accumulator
            uint8_t* stage = staging_ptr + static_cast<size_t>(ew) * g.pack_stage_bytes;
            const int n = static_cast<int>(g.N);
            uint32_t uses = 0;
            bool ok = true;
            for (uint64_t t = blockIdx.x + static_cast<uint64_t>(buf) * gridDim.x; ok && t < g.total_tiles; t += 2 * gridDim.x, ++uses) {
                int batch, mt, nt;
                tile_coords(static_cast<uint32_t>(t), g.m_tiles, g.n_tiles, batch, mt, nt);
                if (!mbar_wait(accf0 + 8 * buf, uses & 1, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const int64_t row0 = static_cast<int64_t>(mt) * BM + quarter * 32;
                const int rows = static_cast<int>(min(static_cast<int64_t>(32), g.M - row0));
                if (rows > 0) {  // warp-uniform
                    float bias = 0.0f;
                    if (g.bias != nullptr && lane < rows)
                        bias = g.is_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(g.bias)[row0 + lane])
                                         : __half2float(static_cast<const __half*>(g.bias)[row0 + lane]);
                    if (lane == 0) bulk_wait_read_0();  // the previous tile's bulk store has read the staging block
                    __syncwarp();
                    uint8_t* gptr = static_cast<uint8_t*>(g.d) + (static_cast<size_t>(batch) * g.d_batch + static_cast<size_t>(row0) * n) * 2;
                    const uint32_t taddr0 = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * BN;
                    const StatsOut so = {g.stat_max, g.stat_sum, g.stat_argmax};
                    drain_packed<typename out_type<OUT>::type, SCALE, PACK == PACK_STATS>(stage, gptr, n, rows, taddr0, g.bias != nullptr, bias, g.scale, lane,
                                                                                          so, static_cast<int64_t>(batch) * g.M + row0);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(acce0 + 8 * buf);
            }
            if (lane == 0) bulk_wait_all();  // shared memory stays valid until the last store has left
        }
    } else if (warp - 2 < g.epi_warps) {
        // ------------------------------------------------------------ epilogue --------
        const int ew = warp - 2;                 // staging slot
        const int quarter = warp & 3;            // TMEM lanes [32*quarter, 32*quarter+32)
        uint8_t* stage = staging_ptr + ew * STAGING_WARP_BYTES;
        uint32_t local_tile = 0;
        int flip = 0;  // which of the warp's two store boxes is next
        bool ok = true;
        for (uint32_t t = blockIdx.x; ok && t < g.total_tiles; t += gridDim.x, ++local_tile) {
            int batch, mt, nt;
            tile_coords(t, g.m_tiles, g.n_tiles, batch, mt, nt);
            const int buf = local_tile & 1;
            const uint32_t parity = (local_tile >> 1) & 1;
            if (!mbar_wait(accf0 + 8 * buf, parity, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const int64_t row0 = static_cast<int64_t>(mt) * BM + quarter * 32;
            const int64_t col_base = static_cast<int64_t>(nt) * g.tile_n;
            const int64_t col_end = min(g.N, col_base + g.tile_n);  // first column this tile does not own
            const uint32_t taddr0 = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * BN;
            float bias = 0.0f;
            if (g.bias != nullptr && row0 + lane < g.M) {
                bias = g.is_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(g.bias)[row0 + lane])
                                 : __half2float(static_cast<const __half*>(g.bias)[row0 + lane]);
            }
            EpilogueTile e;
            e.dbase = static_cast<uint8_t*>(g.d) + static_cast<size_t>(batch) * g.d_batch * (OUT == OUT_F32 ? 4 : 2);
            e.ldd = g.ldd;
            e.row0 = row0;
            e.rows = static_cast<int>(min(static_cast<int64_t>(32), g.M - row0));
            e.col_base = col_base;
            e.col_end = col_end;
            e.taddr0 = taddr0;
            e.chunk0 = ew >> 2;
            e.chunk_step = g.epi_warps >> 2;
            e.bias = bias;
            e.scale = g.scale;
            e.vec_store = g.vec_store;
            e.has_bias = g.bias != nullptr;
            e.tma_store = g.tma_store;
            e.batch = batch;
            e.n_total = g.N;
            e.map_d = &map_d;
            e.mirrors = g.mirror;
            e.n_mirrors = g.n_mirrors;
            e.batch_elems = static_cast<int64_t>(batch) * g.d_batch;
            drain_tile<typename out_type<OUT>::type, SCALE>(e, stage, lane, flip);
            // this warp has finished reading the accumulator
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acce0 + 8 * buf);
        }
        if (g.tma_store && lane == 0) bulk_wait_all();  // shared memory stays valid until the last box has left
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 2) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0 && *abort_flag) atomicAdd(&g_tc_aborts, 1u);
}

// ---- stationary A for short K ---------------------------------------------------------------
// With K <= 256 a tile is one pass of at most four K-blocks, so the ring above holds exactly one
// tile's operands: a stage is refilled only after its MMAs have run, the next tile's first block
// lands one load latency later, and the time per tile is that round trip however little of
// HBM, L2 or the tensor pipe is in use. (Keeping A resident in SHARED memory changes nothing:
// the ring that is left still holds one tile of B. Measured both ways.) This variant takes A
// out of shared memory altogether. A CTA owns ONE 128-row tile of A for its whole life and
// holds it in tensor memory (128 lanes x 128 columns of packed 16-bit pairs, next to two
// 192-column accumulators: 2 * 192 + 128 = 512 columns), the MMAs take A from there
// (tcgen05.mma with a tensor-memory A operand), and all of the ring carries B: eight stages of
// 64 k-rows x 192 columns, i.e. two tiles in flight, with two thirds of the bytes per result
// column. CTAs come in groups that contain every row tile once; the groups split the column
// tiles (over all batches) evenly and the CTAs of a group walk the same columns at about the
// same time, so B is read from HBM once and from L2 by the others. B is N-major ([K, N]: plain
// matmul, the 1x1 convolution on NCHW). Narrower tiles do not pay: an MMA of N = 128 takes
// nearly as long as one of N = 192 when it accumulates into the same columns as the one before
// it (measured: 88 ns against 98 ns), so a variant with two row tiles per CTA and 128-column
// accumulators lost more in the tensor pipe than it saved in L2 traffic.
constexpr int SN = 192;                              // result columns per tile
constexpr int S_STAGES = 8;
constexpr uint32_t S_STAGE_BYTES = SN * BK * 2;      // 24 KiB
constexpr int S_KMAX = 256;
constexpr uint32_t S_A_COL = 2 * SN;                 // first tensor-memory column of A
static_assert(S_STAGES * S_STAGE_BYTES == STAGES * STAGE_BYTES, "the stationary variant reuses the ring's memory");
static_assert(S_A_COL + S_KMAX / 2 <= TMEM_COLS, "two accumulators and A must fit tensor memory");

template <int OUT, bool SCALE>
__global__ void __launch_bounds__(kThreads, 1)
tc_gemm_stationary_kernel(const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_d, const KernelArgs g) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - raw);
    const uint32_t staging = base + S_STAGES * S_STAGE_BYTES;
    uint8_t* staging_ptr = base_ptr + S_STAGES * S_STAGE_BYTES;
    const uint32_t bars = staging + STAGING_BYTES;
    // barrier layout (8 bytes each): full[S_STAGES], empty[S_STAGES], acc_full[2], acc_empty[2]
    const uint32_t full0 = bars, empty0 = bars + 8 * S_STAGES, accf0 = bars + 16 * S_STAGES, acce0 = accf0 + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + S_STAGES * S_STAGE_BYTES + STAGING_BYTES + 16 * S_STAGES + 32);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_blocks = g.k_blocks;
    const int mt = static_cast<int>(blockIdx.x) % g.m_tiles, group = static_cast<int>(blockIdx.x) / g.m_tiles;
    // this group's share of the column tiles
    const uint32_t j0 = static_cast<uint32_t>(static_cast<uint64_t>(group) * g.col_tiles / g.groups);
    const uint32_t j1 = static_cast<uint32_t>(static_cast<uint64_t>(group + 1) * g.col_tiles / g.groups);

    if (threadIdx.x == 0) {
        for (int s = 0; s < S_STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(accf0 + 8 * b, 1);
            mbar_init(acce0 + 8 * b, g.epi_warps);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 2) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp >= 2) {
        // A -> tensor memory: the lane's row, 128 of its K elements per warp (warps 2-5 the first
        // 128, warps 6-9 the rest), zero beyond M and K so that nothing undefined meets the
        // zero-filled rows of B. Rows are read with 16-byte loads straight from global memory: 64 KiB
        // per CTA, once.
        const int quarter = warp & 3, half = (warp - 2) >> 2;
        const int64_t row = static_cast<int64_t>(mt) * BM + quarter * 32 + lane;
        const uint16_t* arow = static_cast<const uint16_t*>(g.a) + row * g.lda;
#pragma unroll 1
        for (int q = 0; q < 2; ++q) {
            const int col0 = half * 64 + q * 32;  // packed columns [col0, col0 + 32) = K elements [2 col0, 2 col0 + 64)
            uint32_t v[32];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int k = 2 * col0 + 8 * u;
                uint4 w = make_uint4(0u, 0u, 0u, 0u);
                if (row < g.M && k < g.k_total) w = __ldg(reinterpret_cast<const uint4*>(arow + k));
                v[4 * u] = w.x; v[4 * u + 1] = w.y; v[4 * u + 2] = w.z; v[4 * u + 3] = w.w;
                if (k + 8 > g.k_total) {  // the row's pitch covers the 16 bytes, K does not: drop what lies past K
#pragma unroll
                    for (int e2 = 0; e2 < 4; ++e2) {
                        const int first = k + 2 * e2;
                        if (first >= g.k_total) v[4 * u + e2] = 0u;
                        else if (first + 1 >= g.k_total) v[4 * u + e2] &= 0xFFFFu;
                    }
                }
            }
            tmem_store(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + S_A_COL + col0, v);
        }
        tmem_store_wait();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer ----
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (uint32_t j = j0; ok && j < j1; ++j) {
                const int batch = static_cast<int>(j / static_cast<uint32_t>(g.n_tiles));
                const int nt = static_cast<int>(j - static_cast<uint32_t>(batch) * static_cast<uint32_t>(g.n_tiles));
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % S_STAGES;
                    const uint32_t parity = ((it / S_STAGES) & 1) ^ 1;
                    if (!mbar_wait(empty0 + 8 * s, parity, abort_flag)) { ok = false; break; }
                    const uint32_t sb = base + s * S_STAGE_BYTES;
                    mbar_expect_tx(full0 + 8 * s, S_STAGE_BYTES);
                    // three boxes of 64 columns x BK rows, 8 KiB each; a box past the last column is zero fill
#pragma unroll
                    for (int c = 0; c < SN / 64; ++c)
                        tma_load_3d(sb + c * (64 * BK * 2), &map_b, full0 + 8 * s, nt * SN + c * 64, kb * BK, g.b_batched ? batch : 0);
                }
            }
            if (!ok) {
                for (int spin = 0; spin < 4096; ++spin) __nanosleep(64);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer ------
        if (lane == 0) {
            const uint32_t fmt = g.is_bf16 ? 1u : 0u;
            const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 16) | (static_cast<uint32_t>(SN >> 3) << 17) |
                                   (static_cast<uint32_t>(BM >> 4) << 24);
            uint32_t it = 0, local_tile = 0;
            bool ok = true;
            for (uint32_t j = j0; ok && j < j1; ++j, ++local_tile) {
                const int buf = local_tile & 1;
                const uint32_t acc_parity = ((local_tile >> 1) & 1) ^ 1;
                if (!mbar_wait(acce0 + 8 * buf, acc_parity, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t tmem_acc = tmem_base + buf * SN;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % S_STAGES;
                    const uint32_t parity = (it / S_STAGES) & 1;
                    if (!mbar_wait(full0 + 8 * s, parity, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sb = base + s * S_STAGE_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        const uint64_t db = smem_desc(sb + k * UMMA_K * 128, 64 * BK * 2, 1024);
                        umma_f16_a_tmem(tmem_acc, tmem_base + S_A_COL + kb * (BK / 2) + k * (UMMA_K / 2), db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(empty0 + 8 * s);
                }
                if (ok) umma_commit(accf0 + 8 * buf);
            }
        }
    } else if (warp - 2 < g.epi_warps) {
        // ------------------------------------------------------------ epilogue --------
        const int ew = warp - 2;
        const int quarter = warp & 3;
        uint8_t* stage = staging_ptr + ew * STAGING_WARP_BYTES;
        uint32_t local_tile = 0;
        int flip = 0;
        bool ok = true;
        const int64_t row0 = static_cast<int64_t>(mt) * BM + quarter * 32;
        float bias = 0.0f;
        if (g.bias != nullptr && row0 + lane < g.M) {
            bias = g.is_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(g.bias)[row0 + lane])
                             : __half2float(static_cast<const __half*>(g.bias)[row0 + lane]);
        }
        for (uint32_t j = j0; ok && j < j1; ++j, ++local_tile) {
            const int batch = static_cast<int>(j / static_cast<uint32_t>(g.n_tiles));
            const int nt = static_cast<int>(j - static_cast<uint32_t>(batch) * static_cast<uint32_t>(g.n_tiles));
            const int buf = local_tile & 1;
            const uint32_t parity = (local_tile >> 1) & 1;
            if (!mbar_wait(accf0 + 8 * buf, parity, abort_flag)) { ok = false; break; }
            tc_fence_after();
            EpilogueTile e;
            e.dbase = static_cast<uint8_t*>(g.d) + static_cast<size_t>(batch) * g.d_batch * (OUT == OUT_F32 ? 4 : 2);
            e.ldd = g.ldd;
            e.row0 = row0;
            e.rows = static_cast<int>(min(static_cast<int64_t>(32), g.M - row0));
            e.col_base = static_cast<int64_t>(nt) * SN;
            e.col_end = min(g.N, e.col_base + SN);
            e.taddr0 = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * SN;
            e.chunk0 = ew >> 2;
            e.chunk_step = g.epi_warps >> 2;
            e.bias = bias;
            e.scale = g.scale;
            e.vec_store = g.vec_store;
            e.has_bias = g.bias != nullptr;
            e.tma_store = g.tma_store;
            e.batch = batch;
            e.n_total = g.N;
            e.map_d = &map_d;
            e.mirrors = nullptr;
            e.n_mirrors = 0;
            e.batch_elems = 0;
            drain_tile<typename out_type<OUT>::type, SCALE>(e, stage, lane, flip);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acce0 + 8 * buf);
        }
        if (g.tma_store && lane == 0) bulk_wait_all();
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 2) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0 && *abort_flag) atomicAdd(&g_tc_aborts, 1u);
}

// ------------------------------------------------------------------ host --------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

bool mult8(int64_t v) { return (v & 7) == 0; }
bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Tiled map of rank `rank`, zero fill outside the tensor.
tn_status encode_as(CUtensorMap* map, const void* ptr, CUtensorMapDataType type, CUtensorMapSwizzle swizzle, int rank,
                    const cuuint64_t* dims, const cuuint64_t* strides, const cuuint32_t* box, const cuuint32_t* traversal = nullptr) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(TN_ERROR, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    if (traversal)
        for (int i = 0; i < rank; ++i) estr[i] = traversal[i];
    CUresult r = fn(map, type, (cuuint32_t)rank, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(TN_ERROR, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    return TN_SUCCESS;
}

// Operand maps: 16-bit elements, 128-byte swizzle.
tn_status encode(CUtensorMap* map, const void* ptr, bool bf16, int rank, const cuuint64_t* dims, const cuuint64_t* strides,
                 const cuuint32_t* box, const cuuint32_t* traversal = nullptr) {
    return encode_as(map, ptr, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, CU_TENSOR_MAP_SWIZZLE_128B,
                     rank, dims, strides, box, traversal);
}

// Result map (columns, rows, batch) for the epilogue's stores: boxes of 32 rows x 64 bytes, 64-byte
// swizzle. Usable when the base and both pitches are multiples of 16 bytes and every tile starts
// on a 16-byte column boundary.
bool can_tma_store(const void* d, int64_t ldd, int64_t d_batch, int64_t tile_n, bool f32) {
    const int64_t per16 = f32 ? 4 : 8;
    static const bool disabled = getenv("TN_TC_NO_TMA_STORE") != nullptr;
    if (disabled) return false;
    return aligned16(d) && ldd % per16 == 0 && d_batch % per16 == 0 && tile_n % per16 == 0;
}
tn_status make_result_map(CUtensorMap* map, void* d, bool f32, bool bf16, int64_t n, int64_t m, int64_t batches, int64_t ldd, int64_t d_batch) {
    const cuuint64_t es = f32 ? 4 : 2;
    cuuint64_t dims[3] = {(cuuint64_t)n, (cuuint64_t)m, (cuuint64_t)(batches > 0 ? batches : 1)};
    cuuint64_t pitch_batch = (cuuint64_t)(d_batch > 0 ? d_batch : ldd * m) * es;
    cuuint64_t strides[2] = {(cuuint64_t)ldd * es, pitch_batch};
    cuuint32_t box[3] = {(cuuint32_t)(64 / es), 32, 1};
    const CUtensorMapDataType type = f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    return encode_as(map, d, type, CU_TENSOR_MAP_SWIZZLE_64B, 3, dims, strides, box);
}

// 3-D map (inner, rows, batch) over a 16-bit matrix; box = box_inner x box_rows x 1.
tn_status make_map(CUtensorMap* map, const void* ptr, bool bf16, int64_t inner, int64_t rows, int64_t batches,
                   int64_t row_pitch, int64_t batch_pitch, int box_inner, int box_rows) {
    cuuint64_t dims[3] = {(cuuint64_t)inner, (cuuint64_t)rows, (cuuint64_t)(batches > 0 ? batches : 1)};
    // a pitch is irrelevant for an extent of 1 but must still be a non-zero multiple of 16 bytes
    cuuint64_t pitch_rows = (cuuint64_t)row_pitch * 2;
    cuuint64_t pitch_batch = (cuuint64_t)(batch_pitch > 0 ? batch_pitch : row_pitch * rows) * 2;
    if (pitch_rows == 0) pitch_rows = (cuuint64_t)inner * 2;
    if (pitch_batch == 0) pitch_batch = pitch_rows;
    cuuint64_t strides[2] = {pitch_rows, pitch_batch};
    cuuint32_t box[3] = {(cuuint32_t)box_inner, (cuuint32_t)box_rows, 1};
    return encode(map, ptr, bf16, 3, dims, strides, box);
}


// Environment knobs are read once per process (measurement aids; the defaults are the tuned values).
int env_epilogue_warps() {
    static const int value = [] {
        const char* v = getenv("TN_TC_EPILOGUE_WARPS");
        const int n = v ? atoi(v) : 0;
        return (n == 4 || n == 8) ? n : 0;
    }();
    return value;
}

template <int MODE, int OUT, bool SCALE, int PACK>
tn_status launch_one(const CUtensorMap& map_a, const CUtensorMap& map_b, const CUtensorMap& map_d, const KernelArgs& g, cudaStream_t stream) {
    // the opt-in shared-memory size is a per-device attribute of the kernel
    static thread_local int attr_device = -1;
    constexpr bool PACKED = PACK != PACK_NONE;
    constexpr uint32_t kSmemMax = PACKED ? PACKED_SMEM_MAX : SMEM_BYTES;
    int dev = 0;
    TN_CUDA(cudaGetDevice(&dev));
    if (attr_device != dev) {
        TN_CUDA(cudaFuncSetAttribute(tc_gemm_kernel<MODE, OUT, SCALE, PACK>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemMax));
        attr_device = dev;
    }
    const int64_t sms = sm_count() - sm_margin();
    const int grid = (int)(g.total_tiles < sms ? g.total_tiles : sms);
    KernelArgs args = g;
    // A long main loop hides a 4-warp epilogue completely; short ones (HBM-bound shapes) are paced
    // by the epilogue and get all eight warps. The packed epilogue always runs eight.
    args.epi_warps = g.k_blocks >= 16 ? 4 : 8;
    if (env_epilogue_warps()) args.epi_warps = env_epilogue_warps();
    uint32_t smem = SMEM_BYTES;
    if (PACKED) {
        args.epi_warps = 8;
        smem = 1024 + PACKED_STAGES * STAGE_BYTES + kEpilogueWarps * g.pack_stage_bytes + 256;
    }
    tc_gemm_kernel<MODE, OUT, SCALE, PACK><<<grid, kThreads, smem, stream>>>(map_a, map_b, map_d, args);
    g_path_launches[PACK == PACK_NONE ? 0 : PACK == PACK_ROWS ? 1 : 2].fetch_add(1, std::memory_order_relaxed);
    return after_launch("tc_gemm_kernel");
}

template <int MODE, int OUT, int PACK>
tn_status launch_scaled(const CUtensorMap& map_a, const CUtensorMap& map_b, const CUtensorMap& map_d, const KernelArgs& g, cudaStream_t stream) {
    return g.has_scale ? launch_one<MODE, OUT, true, PACK>(map_a, map_b, map_d, g, stream)
                       : launch_one<MODE, OUT, false, PACK>(map_a, map_b, map_d, g, stream);
}

template <int MODE>
tn_status launch(const CUtensorMap& map_a, const CUtensorMap& map_b, const CUtensorMap& map_d, const KernelArgs& g, cudaStream_t stream) {
    if (g.d_is_f32) return launch_scaled<MODE, OUT_F32, PACK_NONE>(map_a, map_b, map_d, g, stream);
    if constexpr (MODE != MODE_CONV) {
        if (g.pack_stage_bytes != 0) {
            if (g.stat_max || g.stat_sum || g.stat_argmax)
                return g.is_bf16 ? launch_scaled<MODE, OUT_BF16, PACK_STATS>(map_a, map_b, map_d, g, stream)
                                 : launch_scaled<MODE, OUT_F16, PACK_STATS>(map_a, map_b, map_d, g, stream);
            return g.is_bf16 ? launch_scaled<MODE, OUT_BF16, PACK_ROWS>(map_a, map_b, map_d, g, stream)
                             : launch_scaled<MODE, OUT_F16, PACK_ROWS>(map_a, map_b, map_d, g, stream);
        }
    }
    return g.is_bf16 ? launch_scaled<MODE, OUT_BF16, PACK_NONE>(map_a, map_b, map_d, g, stream)
                     : launch_scaled<MODE, OUT_F16, PACK_NONE>(map_a, map_b, map_d, g, stream);
}

template <int OUT, bool SCALE>
tn_status launch_stationary_one(const CUtensorMap& map_b, const CUtensorMap& map_d, const KernelArgs& g, cudaStream_t stream) {
    static thread_local int attr_device = -1;
    int dev = 0;
    TN_CUDA(cudaGetDevice(&dev));
    if (attr_device != dev) {
        TN_CUDA(cudaFuncSetAttribute(tc_gemm_stationary_kernel<OUT, SCALE>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        attr_device = dev;
    }
    KernelArgs args = g;
    args.epi_warps = env_epilogue_warps() ? env_epilogue_warps() : 8;
    tc_gemm_stationary_kernel<OUT, SCALE><<<g.groups * g.m_tiles, kThreads, SMEM_BYTES, stream>>>(map_b, map_d, args);
    g_path_launches[3].fetch_add(1, std::memory_order_relaxed);
    return after_launch("tc_gemm_stationary_kernel");
}

template <int OUT>
tn_status launch_stationary_scaled(const CUtensorMap& map_b, const CUtensorMap& map_d, const KernelArgs& g, cudaStream_t stream) {
    return g.has_scale ? launch_stationary_one<OUT, true>(map_b, map_d, g, stream) : launch_stationary_one<OUT, false>(map_b, map_d, g, stream);
}

tn_status launch_stationary(const CUtensorMap& map_b, const CUtensorMap& map_d, const KernelArgs& g, cudaStream_t stream) {
    if (g.d_is_f32) return launch_stationary_scaled<OUT_F32>(map_b, map_d, g, stream);
    return g.is_bf16 ? launch_stationary_scaled<OUT_BF16>(map_b, map_d, g, stream) : launch_stationary_scaled<OUT_F16>(map_b, map_d, g, stream);
}

}  // namespace

bool tc_gemm_eligible(const TcGemm& p) {
    if (p.ab_dtype != TN_FLOAT16 && p.ab_dtype != TN_BFLOAT16) return false;
    if (p.d_dtype != p.ab_dtype && p.d_dtype != TN_FLOAT32) return false;
    if (p.M <= 0 || p.N <= 0 || p.K <= 0 || p.batches <= 0) return false;
    if (!aligned16(p.a) || !aligned16(p.b)) return false;
    if (!mult8(p.lda) || !mult8(p.ldb) || !mult8(p.a_batch) || !mult8(p.b_batch)) return false;
    if (p.lda < p.K) return false;
    if (p.b_n_major ? p.ldb < p.N : p.ldb < p.K) return false;
    // extents must fit the 32-bit coordinates of a tensor map with headroom
    if (p.M >= (int64_t(1) << 31) || p.N >= (int64_t(1) << 31) || p.K >= (int64_t(1) << 31) || p.batches >= (int64_t(1) << 31)) return false;
    const int64_t tiles = ceil_div(p.M, BM) * ceil_div(p.N, BN) * p.batches;
    return tiles < (int64_t(1) << 31);
}

bool tc_gemm_can_fuse_stats(const TcGemm& p) {
    return tc_gemm_eligible(p) && p.d_dtype == p.ab_dtype && p.N <= BN && p.ldd == p.N;
}

static bool can_vector_store(const void* d, int64_t ldd, int64_t d_batch, int64_t n, int64_t tile_n, bool f32) {
    const int64_t per16 = f32 ? 4 : 8;  // elements per 16 bytes
    return aligned16(d) && ldd % per16 == 0 && d_batch % per16 == 0 && n % per16 == 0 && tile_n % per16 == 0;
}

tn_status tc_gemm(const TcGemm& p, cudaStream_t stream) {
    const bool bf16 = p.ab_dtype == TN_BFLOAT16;
    CUtensorMap map_a, map_b;
    TN_TRY(make_map(&map_a, p.a, bf16, p.K, p.M, p.a_batch ? p.batches : 1, p.lda, p.a_batch, BK, BM));
    if (p.b_n_major) TN_TRY(make_map(&map_b, p.b, bf16, p.N, p.K, p.b_batch ? p.batches : 1, p.ldb, p.b_batch, 64, BK));
    else TN_TRY(make_map(&map_b, p.b, bf16, p.K, p.N, p.b_batch ? p.batches : 1, p.ldb, p.b_batch, BK, BN));

    KernelArgs g = {};
    g.d = p.d;
    g.bias = p.bias;
    g.M = p.M;
    g.N = p.N;
    g.ldd = p.ldd;
    g.d_batch = p.d_batch;
    g.m_tiles = (int)ceil_div(p.M, BM);
    g.n_tiles = (int)ceil_div(p.N, BN);
    g.total_tiles = (uint32_t)((int64_t)g.m_tiles * g.n_tiles * p.batches);
    g.k_blocks = (int)ceil_div(p.K, BK);
    g.tile_n = BN;
    g.umma_n = BN;
    g.stage_tx = STAGE_BYTES;
    g.a_batched = p.a_batch != 0;
    g.b_batched = p.b_batch != 0;
    g.is_bf16 = bf16;
    g.d_is_f32 = p.d_dtype == TN_FLOAT32;
    g.vec_store = can_vector_store(p.d, p.ldd, p.d_batch, p.N, BN, g.d_is_f32 != 0);
    g.has_scale = p.has_scale;
    g.scale = p.scale;
    CUtensorMap map_d = map_a;  // placeholder when the result does not leave through TMA
    g.tma_store = can_tma_store(p.d, p.ldd, p.d_batch, BN, g.d_is_f32 != 0);
    if (g.tma_store) TN_TRY(make_result_map(&map_d, p.d, g.d_is_f32 != 0, bf16, p.N, p.M, p.batches, p.ldd, p.d_batch));
    // Rows that follow one another without a gap but are not 16-byte multiples: a tile that spans all
    // columns is one contiguous byte range per 32 rows, which the packed epilogue writes in bulk.
    static const bool no_packed = getenv("TN_TC_NO_PACKED") != nullptr;
    const bool wants_stats = p.stat_max || p.stat_sum || p.stat_argmax;
    const bool can_pack = !g.d_is_f32 && g.n_tiles == 1 && p.ldd == p.N;
    if (wants_stats && !can_pack) return fail(TN_ERROR, "fused row statistics need a dense 16-bit result of at most %d columns", BN);
    if (can_pack && (wants_stats || (!g.tma_store && !g.vec_store && !no_packed))) {
        g.pack_stage_bytes = (uint32_t)((32 * p.N * 2 + 16 + 127) & ~int64_t(127));
        g.tma_store = 0;
        g.stat_max = p.stat_max;
        g.stat_sum = p.stat_sum;
        g.stat_argmax = p.stat_argmax;
    }
    if (p.n_mirrors > 0) {
        // mirrored results leave through the 16-byte store path only
        if (p.n_mirrors > 7) return fail(TN_ERROR, "gemm: at most 7 mirrors");
        if (g.d_is_f32 || !g.vec_store || wants_stats) return fail(TN_ERROR, "gemm: mirrored results need a 16-bit result whose base and pitches are multiples of 16 bytes");
        for (int m = 0; m < p.n_mirrors; ++m) {
            if (!aligned16(p.mirrors[m])) return fail(TN_ERROR, "gemm: mirror %d is not 16-byte aligned", m);
            g.mirror[m] = p.mirrors[m];
        }
        g.n_mirrors = p.n_mirrors;
        g.tma_store = 0;
        g.pack_stage_bytes = 0;
        g.stat_max = g.stat_sum = nullptr;
        g.stat_argmax = nullptr;
        return p.b_n_major ? launch<MODE_N>(map_a, map_b, map_d, g, stream) : launch<MODE_K>(map_a, map_b, map_d, g, stream);
    }
    // Short K with B as [K, N] and one A for all batches: A stays in tensor memory (see the stationary kernel).
    static const bool no_stationary = getenv("TN_TC_NO_STATIONARY") != nullptr;
    if (p.b_n_major && p.K <= S_KMAX && (p.a_batch == 0 || p.batches == 1) && g.pack_stage_bytes == 0 && !no_stationary) {
        const int64_t sms = sm_count() - sm_margin();
        const int64_t n_tiles = ceil_div(p.N, SN), col_tiles = n_tiles * p.batches;
        const int64_t groups = g.m_tiles <= sms ? sms / g.m_tiles : 0;
        // enough column tiles per CTA to pay for loading A (below about forty the general kernel is as
        // fast or faster: measured on the 1x1 convolution with 16, 32 and 64 images), and nearly all SMs in use
        if (groups > 0 && col_tiles >= 40 * groups && groups * g.m_tiles * 10 >= sms * 9 && col_tiles < (int64_t(1) << 31)) {
            g.a = p.a;
            g.lda = p.lda;
            g.k_total = (int)p.K;
            g.groups = (int)groups;
            g.col_tiles = (uint32_t)col_tiles;
            g.n_tiles = (int)n_tiles;
            g.tile_n = SN;
            g.umma_n = SN;
            return launch_stationary(map_b, map_d, g, stream);
        }
    }
    return p.b_n_major ? launch<MODE_N>(map_a, map_b, map_d, g, stream) : launch<MODE_K>(map_a, map_b, map_d, g, stream);
}

bool tc_conv_eligible(const TcConv& p) {
    if (p.dtype != TN_FLOAT16 && p.dtype != TN_BFLOAT16) return false;
    if (p.N <= 0 || p.C <= 0 || p.Cout <= 0 || p.Ho <= 0 || p.Wo <= 0) return false;
    if (!mult8(p.C)) return false;                       // NHWC pixel pitch must be a multiple of 16 bytes
    if (p.stride_h < 1 || p.stride_h > 8 || p.stride_w < 1 || p.stride_w > 8) return false;  // traversal strides of a tensor map
    if (p.Wo * p.stride_w > 256 || p.W > 65535 || p.H > 65535) return false;              // a box spans at most 256 elements
    if (p.Kh * p.Kw > 1024 || p.N >= (int64_t(1) << 31)) return false;
    if (ceil_div(p.Cout, BM) * p.Ho * p.N >= (int64_t(1) << 31)) return false;  // tile index is 32-bit
    return aligned16(p.x_nhwc) && aligned16(p.w_packed);
}

tn_status tc_conv(const TcConv& p, cudaStream_t stream) {
    const bool bf16 = p.dtype == TN_BFLOAT16;
    const int taps = (int)(p.Kh * p.Kw);
    int hbox = (int)(256 / p.Wo);
    if (hbox > p.Ho) hbox = (int)p.Ho;
    if (hbox > 256 / p.stride_h) hbox = (int)(256 / p.stride_h);
    if (hbox < 1) hbox = 1;
    CUtensorMap map_a, map_b;
    // weights [tap][Cout][Cin]
    TN_TRY(make_map(&map_a, p.w_packed, bf16, p.C, p.Cout, taps, p.C, p.Cout * p.C, BK, BM));
    // activation [N][H][W][C]: box = 64 channels x Wout x hbox rows x 1 image
    {
        cuuint64_t dims[4] = {(cuuint64_t)p.C, (cuuint64_t)p.W, (cuuint64_t)p.H, (cuuint64_t)p.N};
        cuuint64_t strides[3] = {(cuuint64_t)p.C * 2, (cuuint64_t)p.W * p.C * 2, (cuuint64_t)p.H * p.W * p.C * 2};
        // a strided convolution reads every stride-th pixel: the map walks W and H with that
        // traversal stride, and a box that is to deliver n elements spans n * stride
        cuuint32_t box[4] = {(cuuint32_t)BK, (cuuint32_t)(p.Wo * p.stride_w), (cuuint32_t)(hbox * p.stride_h), 1};
        cuuint32_t walk[4] = {1, (cuuint32_t)p.stride_w, (cuuint32_t)p.stride_h, 1};
        TN_TRY(encode(&map_b, p.x_nhwc, bf16, 4, dims, strides, box, walk));
    }
    KernelArgs g = {};
    g.d = p.y;
    g.bias = p.bias;
    g.M = p.Cout;
    g.N = p.Ho * p.Wo;
    g.ldd = g.N;
    g.d_batch = p.Cout * g.N;
    g.m_tiles = (int)ceil_div(p.Cout, BM);
    g.n_tiles = (int)ceil_div(p.Ho, hbox);
    g.total_tiles = (uint32_t)((int64_t)g.m_tiles * g.n_tiles * p.N);
    g.cblocks = (int)ceil_div(p.C, BK);
    g.k_blocks = taps * g.cblocks;
    g.tile_n = hbox * (int)p.Wo;
    g.umma_n = (g.tile_n + 15) & ~15;
    g.stage_tx = A_BYTES + (uint32_t)(hbox * p.Wo) * BK * 2;
    g.a_batched = g.b_batched = 1;
    g.is_bf16 = bf16;
    g.d_is_f32 = 0;
    g.vec_store = can_vector_store(p.y, g.ldd, g.d_batch, g.N, g.tile_n, false);
    g.has_scale = 0;
    g.scale = 1.0f;
    g.kw = (int)p.Kw;
    g.pad_h = (int)p.pad_h;
    g.pad_w = (int)p.pad_w;
    g.hbox = hbox;
    g.str_h = (int)p.stride_h;
    CUtensorMap map_d = map_a;
    g.tma_store = can_tma_store(p.y, g.ldd, g.d_batch, g.tile_n, false);
    if (g.tma_store) TN_TRY(make_result_map(&map_d, p.y, false, bf16, g.N, p.Cout, p.N, g.ldd, g.d_batch));
    return launch<MODE_CONV>(map_a, map_b, map_d, g, stream);
}

// One warp waits, with the kernels' own bounded wait, on a barrier that nothing will ever complete:
// the wait runs out after `polls` polls, the abort flag goes up and the error counter is bumped,
// exactly as in a GEMM CTA whose producer never delivers. Nothing faults and nothing hangs; the
// kernel returns after at most polls x 64 ns.
__global__ void __launch_bounds__(32) wait_probe_kernel(uint32_t polls) {
    __shared__ __align__(8) uint64_t barrier;
    __shared__ int abort_flag;
    const uint32_t bar = smem_u32(&barrier);
    if (threadIdx.x == 0) {
        mbar_init(bar, 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    bool ok = true;
    if (threadIdx.x == 0) ok = mbar_wait(bar, 0, &abort_flag, polls);
    __syncwarp();
    if (threadIdx.x == 0 && !ok && abort_flag) atomicAdd(&g_tc_aborts, 1u);
}

tn_status tc_wait_probe(cudaStream_t stream, unsigned int polls) {
    if (polls > kSpinLimit) polls = kSpinLimit;
    wait_probe_kernel<<<1, 32, 0, stream>>>(polls);
    return after_launch("wait_probe_kernel");
}

void tc_path_launches(uint64_t (&out)[4]) {
    for (int i = 0; i < 4; ++i) out[i] = g_path_launches[i].load(std::memory_order_relaxed);
}

tn_status tc_abort_count(unsigned int* count) {
    TN_CUDA(cudaMemcpyFromSymbol(count, g_tc_aborts, sizeof(unsigned int)));
    return TN_SUCCESS;
}

}  // namespace tnb
