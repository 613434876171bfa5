// tn_conv2d / tn_conv2d_bias: NCHW cross-correlation with zero padding. Replaces
// src/cuda/conv2d.cu of the reference (one single-thread block per output element).
//
// Paths:
//   1x1, stride 1, no padding, dense fp16/bf16 tensors -> batched tensor-core GEMM
//        y[n] = W[Cout, Cin] . x[n][Cin, H*W]   (x[n] is an N-major B operand);
//   other fp16/bf16 convolutions (stride 1..8) with Wout * stride <= 256 -> implicit GEMM on
//        the tcgen05 main loop: the activation is first re-laid as NHWC and the weights as
//        [tap][Cout][Cin] in scratch memory (TMA needs the channel axis innermost: a tap shift
//        of one pixel along W would otherwise break its 16-byte start alignment), then every
//        (tap, 64-channel block) is one K step whose B tile is a shifted 4-D TMA box;
//   everything else -> direct SIMT kernel (any dtype, any strides), accumulating in float32
//        for half/float32, float64 for float64 and wrapping int64 for integers.
#include "gemm_tc.cuh"

namespace tnb {
namespace {

constexpr int kThreads = 256;

struct ConvArgs {
    const void* x;
    const void* w;
    const void* bias;
    void* y;
    int dt;
    int64_t N, Cin, H, W, Cout, Kh, Kw, Ho, Wo;
    int64_t pad_h, pad_w, str_h, str_w;
    int64_t xs[4], ws[4], ys[4];
    int64_t bias_stride;
    int64_t total;
};

// Fallback for everything the tensor-core paths do not take (fp32, fp64, integers, odd layouts).
// One thread per output element; threads of a warp share (n, co) almost always, so the weight
// loads are broadcasts and the x loads run along the output row. The taps that fall inside the
// image form a rectangle [kh0, kh1) x [kw0, kw1) that depends only on the output position: it is
// clipped once, and the loops below run over exactly the valid taps with running element offsets
// instead of testing every tap. Terms are added channel by channel, tap row by tap row: the order
// of the CPU reference, so floating-point results differ from it only by fused multiply-adds.
template <typename C>
__global__ void __launch_bounds__(kThreads) conv2d_direct(const __grid_constant__ ConvArgs g) {
    const int64_t step = (int64_t)gridDim.x * kThreads;
    for (int64_t o = (int64_t)blockIdx.x * kThreads + threadIdx.x; o < g.total; o += step) {
        const int64_t row = o / g.Wo, ow = o - row * g.Wo;
        const int64_t plane = row / g.Ho, oh = row - plane * g.Ho;
        const int64_t n = plane / g.Cout, co = plane - n * g.Cout;
        const int64_t top = oh * g.str_h - g.pad_h, left = ow * g.str_w - g.pad_w;  // input position of tap (0, 0)
        const int64_t kh0 = top < 0 ? -top : 0, kh1 = min(g.Kh, g.H - top);
        const int64_t kw0 = left < 0 ? -left : 0, kw1 = min(g.Kw, g.W - left);
        // the bias seeds the accumulator (src/cpu/conv2d.cpp:66-113)
        C acc = g.bias ? load_as<C>(g.bias, g.dt, co * g.bias_stride) : C(0);
        int64_t x_plane = n * g.xs[0] + (top + kh0) * g.xs[2] + (left + kw0) * g.xs[3];
        int64_t w_plane = co * g.ws[0] + kh0 * g.ws[2] + kw0 * g.ws[3];
        for (int64_t ci = 0; ci < g.Cin; ++ci, x_plane += g.xs[1], w_plane += g.ws[1]) {
            int64_t x_row = x_plane, w_row = w_plane;
            for (int64_t kh = kh0; kh < kh1; ++kh, x_row += g.xs[2], w_row += g.ws[2]) {
                int64_t xi = x_row, wi = w_row;
                for (int64_t kw = kw0; kw < kw1; ++kw, xi += g.xs[3], wi += g.ws[3]) {
                    const C xv = load_as<C>(g.x, g.dt, xi);
                    const C wv = load_as<C>(g.w, g.dt, wi);
                    if constexpr (std::is_same<C, int64_t>::value) acc = (int64_t)((uint64_t)acc + (uint64_t)xv * (uint64_t)wv);
                    else acc += xv * wv;
                }
            }
        }
        store_as<C>(g.y, g.dt, n * g.ys[0] + co * g.ys[1] + oh * g.ys[2] + ow * g.ys[3], acc);
    }
}

// x[n, c, h, w] (any strides) -> out[n, h, w, c] with the channel pitch padded to Cp (a multiple of 8,
// the padding zero-filled, so that a pixel is a whole number of 16-byte units for TMA); 64 channels x 64 pixels per CTA through a
// padded shared-memory tile so that both sides are contiguous 128-byte runs per 64 threads.
__global__ void __launch_bounds__(256) nchw_to_nhwc(const uint16_t* __restrict__ x, uint16_t* __restrict__ out, int64_t C, int64_t Cp,
                                                    int64_t H, int64_t W, int64_t xs0, int64_t xs1, int64_t xs2, int64_t xs3) {
    __shared__ uint16_t tile[64][66];
    const int64_t HW = H * W;
    const int64_t p0 = (int64_t)blockIdx.x * 64, c0 = (int64_t)blockIdx.y * 64, n = blockIdx.z;
    {
        const int pl = threadIdx.x & 63, cl = threadIdx.x >> 6;
        const int64_t p = p0 + pl;
        const int64_t h = p / W, w = p - h * W;
#pragma unroll 4
        for (int i = 0; i < 16; ++i) {
            const int64_t c = c0 + cl + 4 * i;
            tile[cl + 4 * i][pl] = (p < HW && c < C) ? x[n * xs0 + c * xs1 + h * xs2 + w * xs3] : (uint16_t)0;
        }
    }
    __syncthreads();
    {
        const int cl = threadIdx.x & 63, pl = threadIdx.x >> 6;
        const int64_t c = c0 + cl;
#pragma unroll 4
        for (int i = 0; i < 16; ++i) {
            const int64_t p = p0 + pl + 4 * i;
            if (p < HW && c < Cp) out[(n * HW + p) * Cp + c] = tile[cl][pl + 4 * i];  // channels C..Cp-1 were staged as zeros
        }
    }
}

// The weight re-layout as a job that rides along with the activation re-layout (the extra z slices of that
// launch do it), so that the convolution's staging is one launch, not two.
struct WeightJob {
    const uint16_t* w;
    uint16_t* out;
    int64_t Cout, Cin, Cp, Kh, Kw, ws0, ws1, ws2, ws3;  // Cp: channel pitch of the packed weights (Cin rounded up to 8, zero-filled)
};
// w[co, ci, kh, kw] (any strides) -> out[kh*Kw + kw][co][ci], `part` of `parts` equal shares of thread blocks
__device__ __forceinline__ void pack_weights_part(const WeightJob& j, int64_t part, int64_t parts) {
    const int64_t total = j.Kh * j.Kw * j.Cout * j.Cp;
    for (int64_t i = part * 256 + threadIdx.x; i < total; i += parts * 256) {
        int64_t rem = i;
        const int64_t ci = rem % j.Cp; rem /= j.Cp;
        const int64_t co = rem % j.Cout; rem /= j.Cout;
        const int64_t kw = rem % j.Kw;
        const int64_t kh = rem / j.Kw;
        j.out[i] = ci < j.Cin ? j.w[co * j.ws0 + ci * j.ws1 + kh * j.ws2 + kw * j.ws3] : (uint16_t)0;
    }
}

// Same re-layout for a dense 16-bit NCHW tensor whose image size H*W is a multiple of 8: both
// global sides move 16 bytes per thread. A 64-channel x 64-pixel tile is held as 64 rows of 32
// words (a word = two neighbouring pixels of one channel). Row r sits at row index
// (r % 8) * 8 + r / 8 and its words are XOR-swizzled by 4 * (r / 8), which makes the 16-byte row
// stores and the per-channel word gathers of the second phase both free of bank conflicts.
__global__ void __launch_bounds__(256) nchw_to_nhwc_vec(const uint16_t* __restrict__ x, uint16_t* __restrict__ out, int64_t C,
                                                        int64_t HW, int64_t images, WeightJob weights) {
    __shared__ __align__(16) uint32_t tile[64 * 32];
    if (blockIdx.z >= images) {  // the extra slices repack the weights
        const int64_t per_slice = (int64_t)gridDim.x * gridDim.y, slices = gridDim.z - images;
        pack_weights_part(weights, (blockIdx.z - images) * per_slice + (int64_t)blockIdx.y * gridDim.x + blockIdx.x, per_slice * slices);
        return;
    }
    const int64_t p0 = (int64_t)blockIdx.x * 64, c0 = (int64_t)blockIdx.y * 64, n = blockIdx.z;
#pragma unroll
    for (int it = 0; it < 2; ++it) {
        const int v = threadIdx.x + it * 256;
        const int r = v >> 3, seg = v & 7;
        const int64_t c = c0 + r, p = p0 + seg * 8;
        uint4 val = make_uint4(0, 0, 0, 0);
        if (c < C && p < HW) val = __ldg(reinterpret_cast<const uint4*>(x + (n * C + c) * HW + p));
        const int rp = (r & 7) * 8 + (r >> 3);
        *reinterpret_cast<uint4*>(&tile[rp * 32 + ((4 * seg) ^ (4 * (r >> 3)))]) = val;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int cseg = lane & 7, pp = 4 * warp + (lane >> 3);  // pixel pair 0..31 of the tile
    uint32_t w[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) w[k] = tile[(k * 8 + cseg) * 32 + (pp ^ (4 * cseg))];
    uint4 even, odd;  // pixel 2*pp takes the low halves, pixel 2*pp+1 the high halves
    even.x = __byte_perm(w[0], w[1], 0x5410); odd.x = __byte_perm(w[0], w[1], 0x7632);
    even.y = __byte_perm(w[2], w[3], 0x5410); odd.y = __byte_perm(w[2], w[3], 0x7632);
    even.z = __byte_perm(w[4], w[5], 0x5410); odd.z = __byte_perm(w[4], w[5], 0x7632);
    even.w = __byte_perm(w[6], w[7], 0x5410); odd.w = __byte_perm(w[6], w[7], 0x7632);
    const int64_t p = p0 + 2 * pp, c = c0 + cseg * 8;
    if (c < C && p < HW) {
        *reinterpret_cast<uint4*>(out + (n * HW + p) * C + c) = even;
        *reinterpret_cast<uint4*>(out + (n * HW + p + 1) * C + c) = odd;  // HW is even
    }
}

// The same re-layout as a launch of its own (activations that need no re-layout, or the element-wise one).
__global__ void __launch_bounds__(256) pack_weights(WeightJob job) { pack_weights_part(job, blockIdx.x, gridDim.x); }

bool dense_nchw(const tn_tensor_t* t) {
    int64_t expect = 1;
    for (int d = 3; d >= 0; --d) {
        if (t->shape.sizes[d] != 1 && t->strides.sizes[d] != expect) return false;
        expect *= (int64_t)t->shape.sizes[d];
    }
    return true;
}

// `prepacked`: weights already in the implicit GEMM's layout (tn_conv2d_pack_weights), or null.
tn_status conv_impl(const tn_tensor_t* x, const tn_tensor_t* w, const tn_tensor_t* bias, tn_tensor_t* y,
                    tn_stream_t stream, const size_t pad[2], const size_t stride[2], const void* prepacked = nullptr) {
    if (!x || !w || !y || !pad || !stride) return fail(TN_ERROR, "null argument");
    // dtypes must match, as in the reference's tables (src/cpu/conv2d.cpp:221-253)
    if (x->dtype != w->dtype || !is_numeric(x->dtype) || y->dtype != x->dtype || (bias && bias->dtype != x->dtype))
        return fail(TN_UNSUPPORTED_DTYPE, "conv2d: dtypes (%d, %d) -> %d unsupported", (int)x->dtype, (int)w->dtype, (int)y->dtype);
    if (x->rank != 4 || w->rank != 4 || y->rank != 4 || (bias && bias->rank != 1))
        return fail(TN_ERROR, "conv2d: expected ranks 4, 4 -> 4 (bias 1)");
    if (stride[0] == 0 || stride[1] == 0) return fail(TN_ERROR, "conv2d: zero stride");
    ConvArgs g;
    g.x = x->address;
    g.w = w->address;
    g.bias = bias ? bias->address : nullptr;
    g.y = y->address;
    g.dt = x->dtype;
    g.N = (int64_t)x->shape.sizes[0];
    g.Cin = (int64_t)x->shape.sizes[1];
    g.H = (int64_t)x->shape.sizes[2];
    g.W = (int64_t)x->shape.sizes[3];
    g.Cout = (int64_t)w->shape.sizes[0];
    g.Kh = (int64_t)w->shape.sizes[2];
    g.Kw = (int64_t)w->shape.sizes[3];
    if ((int64_t)w->shape.sizes[1] != g.Cin) return fail(TN_ERROR, "conv2d: kernel expects %zu input channels, signal has %lld", w->shape.sizes[1], (long long)g.Cin);
    if (bias && (int64_t)bias->shape.sizes[0] != g.Cout) return fail(TN_ERROR, "conv2d: bias length %zu, %lld output channels", bias->shape.sizes[0], (long long)g.Cout);
    g.pad_h = (int64_t)pad[0];
    g.pad_w = (int64_t)pad[1];
    g.str_h = (int64_t)stride[0];
    g.str_w = (int64_t)stride[1];
    if (g.H + 2 * g.pad_h < g.Kh || g.W + 2 * g.pad_w < g.Kw) return fail(TN_ERROR, "conv2d: kernel larger than the padded signal");
    g.Ho = (g.H + 2 * g.pad_h - g.Kh) / g.str_h + 1;  // floor, src/cpu/conv2d.cpp:136-137
    g.Wo = (g.W + 2 * g.pad_w - g.Kw) / g.str_w + 1;
    if ((int64_t)y->shape.sizes[0] != g.N || (int64_t)y->shape.sizes[1] != g.Cout || (int64_t)y->shape.sizes[2] != g.Ho ||
        (int64_t)y->shape.sizes[3] != g.Wo)
        return fail(TN_ERROR, "conv2d: result shape does not match [%lld,%lld,%lld,%lld]", (long long)g.N, (long long)g.Cout, (long long)g.Ho, (long long)g.Wo);
    if (x->environment.kind != TN_DEVICE || w->environment.kind != TN_DEVICE ||
        x->environment.resource.device.id != w->environment.resource.device.id ||
        x->environment.resource.device.id != y->environment.resource.device.id ||
        (bias && (bias->environment.kind != TN_DEVICE || bias->environment.resource.device.id != y->environment.resource.device.id)))
        return fail(TN_INCOMPATIBLE_DEVICES, "operands must live on one device");
    TN_TRY(use_device_of(y));
    for (int d = 0; d < 4; ++d) {
        g.xs[d] = x->strides.sizes[d];
        g.ws[d] = w->strides.sizes[d];
        g.ys[d] = y->strides.sizes[d];
    }
    g.bias_stride = bias ? bias->strides.sizes[0] : 0;
    g.total = g.N * g.Cout * g.Ho * g.Wo;
    if (g.total == 0) return TN_SUCCESS;
    cudaStream_t s = as_cuda(stream);

    if (is_half(g.dt) && g.Kh == 1 && g.Kw == 1 && g.str_h == 1 && g.str_w == 1 && g.pad_h == 0 && g.pad_w == 0 &&
        dense_nchw(x) && dense_nchw(w) && dense_nchw(y) && (!bias || g.bias_stride == 1)) {
        TcGemm p;
        p.a = g.w;
        p.b = g.x;
        p.d = g.y;
        p.bias = g.bias;
        p.ab_dtype = p.d_dtype = g.dt;
        p.M = g.Cout;
        p.N = g.H * g.W;
        p.K = g.Cin;
        p.lda = g.Cin;
        p.ldb = p.N;
        p.ldd = p.N;
        p.batches = g.N;
        p.a_batch = 0;
        p.b_batch = g.Cin * p.N;
        p.d_batch = g.Cout * p.N;
        p.b_n_major = true;
        if (tc_gemm_eligible(p)) return tc_gemm(p, s);
    }

    if (is_half(g.dt) && g.str_h <= 8 && g.str_w <= 8 && dense_nchw(y) && (!bias || g.bias_stride == 1) && g.N <= 65535) {
        TcConv p;
        // a pixel of the NHWC copy must be a whole number of 16-byte units: channel counts that are not a
        // multiple of 8 (a 3-channel stem) are padded with zero channels in the copy and in the packed weights
        const int64_t Cp = (g.Cin + 7) & ~int64_t(7);
        p.bias = g.bias;
        p.y = g.y;
        p.dtype = g.dt;
        p.N = g.N; p.C = Cp; p.H = g.H; p.W = g.W; p.Cout = g.Cout; p.Kh = g.Kh; p.Kw = g.Kw;
        p.Ho = g.Ho; p.Wo = g.Wo; p.pad_h = g.pad_h; p.pad_w = g.pad_w;
        p.stride_h = g.str_h; p.stride_w = g.str_w;
        // placeholders so that the eligibility test sees aligned pointers; the real ones follow
        p.x_nhwc = g.y;
        p.w_packed = g.y;
        if (tc_conv_eligible(p)) {
            // an activation that already lies as [N][H][W][C] in memory (an NCHW view of channels-last
            // storage) is read in place; only the weights are repacked then
            const bool x_is_nhwc = Cp == g.Cin && g.xs[1] == 1 && g.xs[3] == g.Cin && g.xs[2] == g.W * g.Cin && g.xs[0] == g.H * g.W * g.Cin &&
                                   (reinterpret_cast<uintptr_t>(g.x) & 15) == 0;
            if (prepacked != nullptr && (reinterpret_cast<uintptr_t>(prepacked) & 15) != 0) return fail(TN_ERROR, "conv2d: packed weights must be 16-byte aligned");
            const size_t x_bytes = x_is_nhwc ? 0 : (size_t)(g.N * g.H * g.W * Cp) * 2;
            const size_t w_bytes = prepacked ? 0 : (size_t)(g.Kh * g.Kw * g.Cout * Cp) * 2;
            const size_t x_padded = (x_bytes + 255) & ~size_t(255);
            uint8_t* scratch = nullptr;
            if (x_padded + w_bytes > 0) TN_TRY(scratch_alloc(reinterpret_cast<void**>(&scratch), x_padded + w_bytes, s));
            uint16_t* xh = reinterpret_cast<uint16_t*>(scratch);
            uint16_t* wp = prepacked ? const_cast<uint16_t*>(static_cast<const uint16_t*>(prepacked)) : reinterpret_cast<uint16_t*>(scratch + x_padded);
            const dim3 tgrid((unsigned)ceil_div(g.H * g.W, 64), (unsigned)ceil_div(g.Cin, 64), (unsigned)g.N);
            tn_status st = TN_SUCCESS;
            bool weights_packed = prepacked != nullptr;
            const bool vec_staging = !x_is_nhwc && Cp == g.Cin && dense_nchw(x) && (g.H * g.W) % 8 == 0 && (reinterpret_cast<uintptr_t>(g.x) & 15) == 0;
            const WeightJob job{static_cast<const uint16_t*>(g.w), wp, g.Cout, g.Cin, Cp, g.Kh, g.Kw, g.ws[0], g.ws[1], g.ws[2], g.ws[3]};
            if (x_is_nhwc) {
                xh = const_cast<uint16_t*>(static_cast<const uint16_t*>(g.x));
            } else {
                if (vec_staging) {
                    // one launch for both re-layouts: the weights ride along in one extra z slice (none when they came packed)
                    const dim3 both(tgrid.x, tgrid.y, tgrid.z + (prepacked ? 0 : 1));
                    nchw_to_nhwc_vec<<<both, 256, 0, s>>>(static_cast<const uint16_t*>(g.x), xh, g.Cin, g.H * g.W, g.N, job);
                    weights_packed = true;
                } else {
                    nchw_to_nhwc<<<tgrid, 256, 0, s>>>(static_cast<const uint16_t*>(g.x), xh, g.Cin, Cp, g.H, g.W, g.xs[0], g.xs[1], g.xs[2], g.xs[3]);
                }
                st = after_launch("nchw_to_nhwc");
            }
            if (st == TN_SUCCESS && !weights_packed) {
                int64_t wblocks = ceil_div(g.Kh * g.Kw * g.Cout * Cp, 256);
                if (wblocks > 1184) wblocks = 1184;
                pack_weights<<<(unsigned)wblocks, 256, 0, s>>>(job);
                st = after_launch("pack_weights");
            }
            if (st == TN_SUCCESS) {
                p.x_nhwc = xh;
                p.w_packed = wp;
                st = tc_conv(p, s);
            }
            const tn_status fr = scratch ? scratch_free(scratch, s) : TN_SUCCESS;
            return st != TN_SUCCESS ? st : fr;
        }
    }

    const int64_t cap = (int64_t)sm_count() * 8;
    int64_t blocks = ceil_div(g.total, kThreads);
    if (blocks > cap) blocks = cap;
    if (g.dt == TN_FLOAT64) conv2d_direct<double><<<(int)blocks, kThreads, 0, s>>>(g);
    else if (is_float(g.dt)) conv2d_direct<float><<<(int)blocks, kThreads, 0, s>>>(g);
    else conv2d_direct<int64_t><<<(int)blocks, kThreads, 0, s>>>(g);
    return after_launch("conv2d_direct");
}

}  // namespace
}  // namespace tnb

using namespace tnb;

extern "C" {

tn_status tn_conv2d(const tn_tensor_t* x, const tn_tensor_t* w, tn_tensor_t* y, tn_stream_t stream, const size_t pad[2],
                    const size_t stride[2]) {
    return conv_impl(x, w, nullptr, y, stream, pad, stride);
}

// Weights in the layout the implicit GEMM reads: [tap][Cout][Cin rounded up to 8], zero-filled padding.
static bool packable(const tn_tensor_t* w) { return w && w->rank == 4 && is_half(w->dtype); }

tn_status tn_conv2d_packed_weights_size(const tn_tensor_t* w, size_t* nbytes) {
    if (!w || !nbytes) return fail(TN_ERROR, "null argument");
    if (w->rank != 4) return fail(TN_ERROR, "conv2d: expected weights of rank 4");
    const size_t cp = (w->shape.sizes[1] + 7) & ~size_t(7);
    *nbytes = packable(w) ? w->shape.sizes[2] * w->shape.sizes[3] * w->shape.sizes[0] * cp * 2 : 0;
    return TN_SUCCESS;
}

tn_status tn_conv2d_pack_weights(const tn_tensor_t* w, void* packed, tn_stream_t stream) {
    if (!w || !packed) return fail(TN_ERROR, "null argument");
    if (!packable(w)) return fail(TN_UNSUPPORTED_DTYPE, "conv2d: only float16 / bfloat16 weights of rank 4 have a packed form");
    if ((reinterpret_cast<uintptr_t>(packed) & 15) != 0) return fail(TN_ERROR, "conv2d: packed weights must be 16-byte aligned");
    TN_TRY(use_device_of(w));
    const int64_t cout = w->shape.sizes[0], cin = w->shape.sizes[1], kh = w->shape.sizes[2], kw = w->shape.sizes[3];
    const int64_t cp = (cin + 7) & ~int64_t(7);
    if (cout * cp * kh * kw == 0) return TN_SUCCESS;
    const WeightJob job{static_cast<const uint16_t*>(w->address), static_cast<uint16_t*>(packed), cout, cin, cp, kh, kw,
                        w->strides.sizes[0], w->strides.sizes[1], w->strides.sizes[2], w->strides.sizes[3]};
    int64_t blocks = ceil_div(kh * kw * cout * cp, 256);
    if (blocks > 1184) blocks = 1184;
    pack_weights<<<(unsigned)blocks, 256, 0, as_cuda(stream)>>>(job);
    return after_launch("pack_weights");
}

tn_status tn_conv2d_prepacked(const tn_tensor_t* x, const tn_tensor_t* w, const void* packed, const tn_tensor_t* bias, tn_tensor_t* y,
                              tn_stream_t stream, const size_t pad[2], const size_t stride[2]) {
    return conv_impl(x, w, bias, y, stream, pad, stride, packed);
}

// 1-D convolution as the H = 1 case of conv2d: [N, C, L] * [Cout, Cin, K] -> [N, Cout, Lout].
tn_status tn_conv1d(const tn_tensor_t* x, const tn_tensor_t* w, tn_tensor_t* y, tn_stream_t stream, size_t pad, size_t stride) {
    if (!x || !w || !y) return fail(TN_ERROR, "null argument");
    if (x->rank != 3 || w->rank != 3 || y->rank != 3) return fail(TN_ERROR, "conv1d: expected ranks 3, 3 -> 3");
    auto lift = [](const tn_tensor_t* t) {
        tn_tensor_t r = *t;
        r.rank = 4;
        r.shape.sizes[3] = t->shape.sizes[2];
        r.strides.sizes[3] = t->strides.sizes[2];
        r.shape.sizes[2] = 1;
        r.strides.sizes[2] = (int64_t)t->shape.sizes[2] * t->strides.sizes[2];
        return r;
    };
    const tn_tensor_t x4 = lift(x), w4 = lift(w);
    tn_tensor_t y4 = lift(y);
    const size_t pad2[2] = {0, pad}, stride2[2] = {1, stride};
    return conv_impl(&x4, &w4, nullptr, &y4, stream, pad2, stride2);
}

tn_status tn_conv2d_bias(const tn_tensor_t* x, const tn_tensor_t* w, const tn_tensor_t* bias, tn_tensor_t* y,
                         tn_stream_t stream, const size_t pad[2], const size_t stride[2]) {
    if (!bias) return fail(TN_ERROR, "null bias");
    return conv_impl(x, w, bias, y, stream, pad, stride);
}

}  // extern "C"
