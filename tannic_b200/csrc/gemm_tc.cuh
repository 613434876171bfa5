// Interface between the GEMM / conv dispatchers and the tcgen05 tensor-core kernel.
#pragma once

#include "common.cuh"

namespace tnb {

// One batched GEMM  D[b] = A[b] . B[b]^T-or-not  on 16-bit operands with fp32 accumulation in
// TMEM. A is K-major ([M, K], K contiguous). B is K-major ([N, K], K contiguous: the layout of
// `W` in `matmul(X, W.transpose(-1,-2))`) or N-major ([K, N], N contiguous: plain matmul, and
// the activation matrix [Cin, H*W] of a 1x1 convolution).
struct TcGemm {
    const void* a = nullptr;
    const void* b = nullptr;
    void* d = nullptr;
    const void* bias = nullptr;  // optional per-row (M) bias of the operand dtype, seeds the accumulator
    int ab_dtype = 0;            // TN_FLOAT16 or TN_BFLOAT16
    int d_dtype = 0;             // ab_dtype or TN_FLOAT32
    int64_t M = 0, N = 0, K = 0;
    int64_t lda = 0, ldb = 0, ldd = 0;              // leading dimensions in elements
    int64_t batches = 1;
    int64_t a_batch = 0, b_batch = 0, d_batch = 0;  // batch strides in elements, 0 = shared
    bool b_n_major = false;
    bool has_scale = false;      // d = round(round(acc) * scale)
    float scale = 1.0f;
    // Optional fused row statistics of the (rounded, scaled) result along its last axis, indexed by
    // batch * M + row; usable when tc_gemm_can_fuse_stats(p). Value outputs have the result's dtype.
    // Further result buffers of the same shape, dtype and pitches (memory of other GPUs mapped into this
    // process): every tile is written into each of them as well, by plain 16-byte stores from the epilogue.
    void* mirrors[7] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    int n_mirrors = 0;
    void* stat_max = nullptr;
    void* stat_sum = nullptr;
    int64_t* stat_argmax = nullptr;
};
// True when the result is 16-bit, dense (ldd == N) and one tile wide (N <= 256): then each result row
// is drained by one thread, which can keep the row's maximum, sum and argmax as it goes.
bool tc_gemm_can_fuse_stats(const TcGemm& p);

// Implicit-GEMM convolution (stride 1) on the same main loop. `x_nhwc` is the activation in
// [N, H, W, C] order and `w_packed` the weights in [Kh*Kw, Cout, Cin] order (both produced by the
// caller in scratch memory); the result is written as dense NCHW.
struct TcConv {
    const void* x_nhwc = nullptr;
    const void* w_packed = nullptr;
    const void* bias = nullptr;  // optional [Cout]
    void* y = nullptr;
    int dtype = 0;
    int64_t N = 0, C = 0, H = 0, W = 0, Cout = 0, Kh = 0, Kw = 0, Ho = 0, Wo = 0, pad_h = 0, pad_w = 0;
    int64_t stride_h = 1, stride_w = 1;  // 1..8: the traversal strides of the activation's tensor map
};
bool tc_conv_eligible(const TcConv& p);
tn_status tc_conv(const TcConv& p, cudaStream_t stream);

// True when TMA can address the operands (16-byte aligned bases and pitches).
bool tc_gemm_eligible(const TcGemm& p);
tn_status tc_gemm(const TcGemm& p, cudaStream_t stream);

}  // namespace tnb
