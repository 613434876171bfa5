/*
 * tannic_b200.h — C ABI of the B200 (sm_100a) device backend for Tannic's operator core.
 *
 * Every entry point is `extern "C"`, takes plain records / pointers / sizes and returns a
 * tn_status. The records below are layout-identical to the reference's own runtime PODs
 * (include/tannic/runtime/tensor.h:37-73, types.h:29-44, status.h:26-32, streams.h:32-37,
 * resources.h:35-59), so a `tannic::tensor_t*` can be passed where a `tn_tensor_t*` is
 * expected without any marshalling. Each declaration cites the reference symbol it replaces.
 *
 * Conventions shared by all ops (reference include/tannic/callback.hpp:36-180):
 *   - the caller owns every tensor; `dst` is allocated by the caller before the call with
 *     `tn_dtype_size(dst->dtype) * dst->size` bytes and is written densely in logical
 *     row-major order (its strides are read only by gemm / conv2d / cpy, as in the reference);
 *   - `address` already contains the view's byte offset; strides are in ELEMENTS;
 *   - ops are asynchronous on the stream passed in; `stream.address == 0` is the legacy
 *     default stream;
 *   - an op never allocates user-visible memory; scratch comes from the backend's own
 *     stream-ordered pool;
 *   - there is no CPU fallback: every failure is reported as a status, never by exit().
 */
#ifndef TANNIC_B200_H
#define TANNIC_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TN_MAX_RANK 8

/* reference: enum type, include/tannic/runtime/types.h:29-44 (same order, same values) */
typedef enum tn_dtype {
    TN_ANY = 0,
    TN_BOOLEAN,
    TN_INT8,
    TN_INT16,
    TN_INT32,
    TN_INT64,
    TN_FLOAT16,
    TN_BFLOAT16,
    TN_FLOAT32,
    TN_FLOAT64,
    TN_COMPLEX64,
    TN_COMPLEX128,
    TN_UNKNOWN,
    TN_TYPES
} tn_dtype;

/* reference: enum status, include/tannic/runtime/status.h:26-32 */
typedef enum tn_status {
    TN_SUCCESS = 0,
    TN_ERROR,
    TN_UNSUPPORTED_DTYPE,
    TN_NULL_ALLOCATOR,
    TN_INCOMPATIBLE_DEVICES
} tn_status;

/* reference: enum layout, include/tannic/runtime/tensor.h:37-41 */
typedef enum tn_layout { TN_SINGLETON = 0, TN_CONTIGUOUS, TN_STRIDED } tn_layout;

/* reference: environment / host / device records, include/tannic/runtime/resources.h:35-59 */
typedef enum tn_environment_kind { TN_HOST = 0, TN_DEVICE } tn_environment_kind;
typedef enum tn_host_traits { TN_PAGEABLE = 1 << 0, TN_PINNED = 1 << 1 } tn_host_traits;
typedef struct tn_host_t { tn_host_traits traits; } tn_host_t;
typedef struct tn_device_t { int id; } tn_device_t;
typedef struct tn_environment_t {
    tn_environment_kind kind;
    union {
        tn_host_t host;
        tn_device_t device;
    } resource;
} tn_environment_t;

/* reference: scalar_t / shape_t / strides_t / tensor_t, include/tannic/runtime/tensor.h:43-73 */
typedef struct tn_scalar_t {
    const void* address;
    tn_dtype dtype;
} tn_scalar_t;

typedef struct tn_shape_t {
    union {
        const size_t* address;
        size_t sizes[TN_MAX_RANK];
    };
} tn_shape_t;

typedef struct tn_strides_t {
    union {
        const int64_t* address;
        int64_t sizes[TN_MAX_RANK];
    };
} tn_strides_t;

typedef struct tn_tensor_t {
    void* address;            /* first logical element (view offset already applied)   */
    uint8_t rank;             /* 0..8                                                   */
    tn_shape_t shape;         /* extents                                                */
    tn_strides_t strides;     /* element strides                                        */
    tn_dtype dtype;
    tn_environment_t environment;
    size_t size;              /* logical element count                                  */
    tn_layout layout;         /* hint computed by the front-end from the strides        */
} tn_tensor_t;

/* reference: stream_t, include/tannic/runtime/streams.h:32-34 (a cudaStream_t as integer) */
typedef struct tn_stream_t { uintptr_t address; } tn_stream_t;

/* ------------------------------------------------------------------ runtime ---------- */

/* Bytes per element of a dtype (0 for any/unknown). reference: dsizeof, include/tannic/types.hpp */
size_t tn_dtype_size(tn_dtype dtype);
/* Text of the most recent failure on the calling thread ("" if none). No reference counterpart:
 * the reference prints and calls exit() (src/cuda/exc.cuh:8-16). */
const char* tn_last_error(void);

/* reference: cuda::getDeviceCount / cuda::setDevice, src/cuda/mem.cu:9-17 */
tn_status tn_device_count(int* count);
tn_status tn_set_device(int id);

/* reference: cuda::Streams::pop / put behind tannic::pop_stream / put_stream,
 * src/cuda/streams.cu:23-38, src/bindings.cpp:22-42. Streams are handed out in LIFO order, so
 * successive ops of one thread land on one stream and are ordered; they are created like the
 * reference's (cudaStreamCreate: ordered with the legacy default stream); the pool is
 * mutex-protected. tn_stream_synchronize returns TN_ERROR (with text) when a thread block gave up
 * on a bounded device-side wait since the last synchronising call on that device. */
tn_status tn_stream_pop(const tn_device_t* device, tn_stream_t* stream);
tn_status tn_stream_put(const tn_device_t* device, tn_stream_t stream);
tn_status tn_stream_synchronize(tn_stream_t stream);

/* reference: cuda::allocate / cuda::deallocate, src/cuda/mem.cu:19-36. Stream-ordered allocation
 * from a memory pool that belongs to this library (one per device, release threshold = unlimited so
 * freed blocks are reused without returning to the driver; the process-wide default pool is left
 * alone). Allocation and release are ordered on the device's pool stream, and through it with the
 * legacy default stream; a caller that uses the memory on another non-blocking stream orders that
 * stream itself. A failed allocation returns TN_ERROR with *address = NULL; the process goes on. */
tn_status tn_allocate(const tn_device_t* device, size_t nbytes, void** address);
tn_status tn_deallocate(const tn_device_t* device, void* address);

/* reference: cuda::copyFromHost / copyDeviceToHost / compareFromHost, src/cuda/mem.cu:38-65.
 * tn_copy_from_host returns once the copy is queued on the pool stream: a pageable source may be
 * reused at once, a pinned one must stay unchanged until that stream has passed the copy.
 * tn_copy_to_host waits for the copy and, like tn_stream_synchronize, reports device-side aborts. */
tn_status tn_copy_from_host(const tn_device_t* device, const void* host, void* dev, size_t nbytes);
tn_status tn_copy_to_host(const tn_device_t* device, const void* dev, void* host, size_t nbytes);
tn_status tn_compare_from_host(const tn_device_t* device, const void* host, const void* dev,
                               size_t nbytes, int* equal);
/* Bulk initialisation. The front-end fills a device tensor from an initializer list with one
 * cuda::copyFromHost of dsizeof(dtype) bytes per element (Tensor::assign, src/tensor.cpp:34-44).
 * tn_assign_from_host takes the place of that call for small writes: writes that extend one
 * contiguous device range are gathered on the calling thread and leave as ONE copy when the range
 * is broken, when 4 MiB have gathered, or when the thread enters any other entry point of this
 * library (each flushes first, so the order of a thread's calls is kept). tn_flush_assignments
 * sends what is pending now; call it before handing the memory to code outside this library.
 * tn_h2d_copy_count counts the host-to-device copies issued by tn_copy_from_host and by these
 * flushes since load (a test aid). */
tn_status tn_assign_from_host(const tn_device_t* device, const void* host, void* dev, size_t nbytes);
tn_status tn_flush_assignments(void);
uint64_t tn_h2d_copy_count(void);
/* Stream-ordered variants with no reference counterpart (the reference copies synchronously): they
 * return once the copy is queued on `stream`; the host range should come from
 * tn_host_allocate_pinned, a pageable one makes the copy synchronous. The caller keeps both ranges
 * alive until the stream has passed the copy. */
tn_status tn_copy_from_host_async(const tn_device_t* device, const void* host, void* dev, size_t nbytes, tn_stream_t stream);
tn_status tn_copy_to_host_async(const tn_device_t* device, const void* dev, void* host, size_t nbytes, tn_stream_t stream);
/* reference: cuda::copy (Tensor::to), src/cuda/mem.cu:67-93 — direction from the two
 * environments; pinned host memory copies asynchronously on `stream`, pageable synchronously. */
tn_status tn_copy(const tn_tensor_t* src, tn_tensor_t* dst, size_t nbytes, tn_stream_t stream);
/* Pinned host memory for the transfer path. The reference's Host(pinned) throws
 * "not supported yet" (src/resources.cpp:24-38). */
tn_status tn_host_allocate_pinned(size_t nbytes, void** address);
tn_status tn_host_free_pinned(void* address);
/* Host-memory placement for the transfer path. No reference counterpart (its `Mesh` of devices is a
 * TODO, include/tannic/resources.hpp:194-197, and nothing there knows which host memory node a GPU
 * hangs off). tn_device_numa_node reports the node of the device's PCIe function (-1 where the
 * platform names none); tn_host_allocate_pinned_near pins memory preferably on that node, or, when the
 * node is unknown and the host has several, interleaved over all of them (freed with
 * tn_host_free_pinned); tn_bind_thread_near restricts the calling thread to that node's CPUs (within
 * the CPUs the process may use). All succeed without effect where the platform gives no information.
 * tn_host_memory_nodes: memory nodes the kernel reports online (0 when it does not say). */
tn_status tn_device_numa_node(const tn_device_t* device, int* node);
int tn_host_memory_nodes(void);
tn_status tn_host_allocate_pinned_near(const tn_device_t* device, size_t nbytes, void** address);
tn_status tn_bind_thread_near(const tn_device_t* device, int* node);

/* ------------------------------------------------------------------ elementwise ------ */

/* reference: cuda::add/sub/mul/pow, src/cuda/ops-binary.cu:485-499 (CPU twin
 * src/cpu/ops-binary.cpp:434-448). NumPy broadcast, operands may be strided views; the result
 * is written in dst->dtype (never wider than the buffer, unlike the reference's half x int
 * and pow(half,half) entries). Arithmetic class: any float64 or (int64 with a float) ->
 * float64; any other float -> float32; integers wrap modulo 2^n. complex64 / complex128 operands
 * of one type support add, sub and mul (and neg / repack below), as in the reference's tables. */
tn_status tn_add(const tn_tensor_t* a, const tn_tensor_t* b, tn_tensor_t* dst, tn_stream_t stream);
tn_status tn_sub(const tn_tensor_t* a, const tn_tensor_t* b, tn_tensor_t* dst, tn_stream_t stream);
tn_status tn_mul(const tn_tensor_t* a, const tn_tensor_t* b, tn_tensor_t* dst, tn_stream_t stream);
tn_status tn_pow(const tn_tensor_t* a, const tn_tensor_t* b, tn_tensor_t* dst, tn_stream_t stream);

/* reference: cuda::neg/repack/log/exp/sqrt/rsqrt/abs/sin/cos/tan/sinh/cosh/tanh,
 * src/cuda/ops-unary.cu:249-444 (CPU twin src/cpu/ops-unary.cpp:202-370). Half types compute in
 * float32 and round once on store; rsqrt(x, eps) = 1/sqrt(x + eps). */
tn_status tn_neg(const tn_tensor_t* src, tn_tensor_t* dst, tn_stream_t stream);
tn_status tn_repack(const tn_tensor_t* src, tn_tensor_t* dst, tn_stream_t stream);
tn_status tn_log(const tn_tensor_t* src, tn_tensor_t* dst, tn_stream_t stream);
tn_status tn_exp(const tn_tensor_t* src, tn_tensor_t* dst, tn_stream_t stream);
tn_status tn_sqrt(const tn_tensor_t* src, tn_tensor_t* dst, tn_stream_t stream);
tn_status tn_rsqrt(const tn_tensor_t* src, tn_tensor_t* dst, tn_stream_t stream, float eps);
tn_status tn_abs(const tn_tensor_t* src, tn_tensor_t* dst, tn_stream_t stream);
tn_status tn_sin(const tn_tensor_t* src, tn_tensor_t* dst, tn_stream_t stream);
tn_status tn_cos(const tn_tensor_t* src, tn_tensor_t* dst, tn_stream_t stream);
tn_status tn_tan(const tn_tensor_t* src, tn_tensor_t* dst, tn_stream_t stream);
tn_status tn_sinh(const tn_tensor_t* src, tn_tensor_t* dst, tn_stream_t stream);
tn_status tn_cosh(const tn_tensor_t* src, tn_tensor_t* dst, tn_stream_t stream);
tn_status tn_tanh(const tn_tensor_t* src, tn_tensor_t* dst, tn_stream_t stream);

/* reference: cuda::scale, src/cuda/ops-scale.cu:126-128 (CPU twin src/cpu/ops-scale.cpp:120-122):
 * dst = src * scalar, scalar dtype must equal the tensor dtype. */
tn_status tn_scale(const tn_tensor_t* src, const tn_scalar_t* scalar, tn_tensor_t* dst,
                   tn_stream_t stream);

/* Fused elementwise program: the whole expression tree in ONE pass over HBM. Replaces the
 * chain of per-node launches and full-size temporaries that Binary<>/Function<>::forward emit
 * (include/tannic/tensor.hpp:351-371, include/tannic/functions.hpp:52-57). Semantics are those
 * of the chain: every node computes in float32 (half types) and is rounded to the storage dtype
 * before the next node reads it. All inputs and dst share one dtype. */
typedef enum tn_eltwise_opcode {
    TN_OP_ADD = 0, TN_OP_SUB, TN_OP_MUL, TN_OP_POW,
    TN_OP_NEG, TN_OP_LOG, TN_OP_EXP, TN_OP_SQRT, TN_OP_RSQRT, TN_OP_ABS,
    TN_OP_SIN, TN_OP_COS, TN_OP_TAN, TN_OP_SINH, TN_OP_COSH, TN_OP_TANH,
    TN_OP_SCALE,
    TN_OP_COUNT
} tn_eltwise_opcode;

#define TN_PROGRAM_MAX_INPUTS 4
#define TN_PROGRAM_MAX_NODES 16

/* Node k produces value (TN_PROGRAM_MAX_INPUTS + k); operands name an input (0..3) or an
 * earlier node's value. The last node is the result. `imm` is eps for RSQRT and the factor
 * for SCALE. */
typedef struct tn_eltwise_node_t {
    uint8_t opcode;
    uint8_t lhs;
    uint8_t rhs;  /* ignored by unary nodes */
    float imm;
} tn_eltwise_node_t;

tn_status tn_eltwise_program(const tn_tensor_t* const* inputs, int n_inputs,
                             const tn_eltwise_node_t* nodes, int n_nodes,
                             tn_tensor_t* dst, tn_stream_t stream);

/* The same program over HOST tensors: dense inputs and a dense result in host memory (pinned memory
 * from tn_host_allocate_pinned[_near] makes the copies asynchronous), evaluated on `device`. The rows
 * (leading extent of dst) are cut into `chunks` pieces (0 = 8) and the copy-in of piece c + 1, the
 * kernel of piece c and the copy-out of piece c - 1 overlap on three private streams; inputs smaller
 * than the result (a broadcast row) are copied whole first. Returns when dst is complete. Device
 * staging memory is kept between calls and only grows. Replaces the reference's sequence of
 * Tensor::to(Device) -> one launch per node -> read-back, each a synchronous cudaMemcpy
 * (src/tensor.cpp:34-136, src/cuda/mem.cu:54-90). Calls on one device are serialised inside the
 * library; calls on different devices (one host thread each) run side by side. */
tn_status tn_eltwise_program_host(const tn_device_t* device, const tn_tensor_t* const* inputs, int n_inputs,
                                  const tn_eltwise_node_t* nodes, int n_nodes, tn_tensor_t* dst, int chunks);

/* Programs that none of the ahead-of-time compiled node lists covers are instantiated at run time:
 * the library hands the text of its own kernel template plus the caller's node list to NVRTC
 * (looked up with dlopen, CUDA headers under CUDA_HOME / CUDA_PATH / /usr/local/cuda), loads the
 * sm_100a image and keeps it for the life of the process, keyed by device, element type, node list
 * and operand kinds; immediates stay arguments. A compilation takes about a second, so by default
 * only results of 2^20 elements and more trigger one. Without NVRTC, or when a compilation fails,
 * the in-kernel interpreter runs the program instead: same results bit for bit, about a third of
 * the speed. The reference has no counterpart (one kernel launch per node, include/tannic/tensor.hpp:351-371).
 * mode: 0 = never compile, 1 = compile for large results (default; TN_PROGRAM_JIT=0 in the
 * environment selects 0), 2 = always compile. */
tn_status tn_program_jit_enable(int mode);
/* Counters since the process started: programs compiled, compilations that failed (those programs are
 * interpreted from then on), whether NVRTC and its headers were found, and programs whose image was read
 * from the disk cache instead of being compiled: when TN_PROGRAM_JIT_CACHE names a directory, compiled images
 * are kept there between processes under a hash of everything they depend on (nothing is written anywhere
 * otherwise). Any pointer may be null. */
tn_status tn_program_jit_stats(unsigned int* compiled, unsigned int* failed, unsigned int* available, unsigned int* from_disk);
/* Compiler output of the last failed compilation (empty when none failed); for diagnostics. */
const char* tn_program_jit_log(void);

/* ------------------------------------------------------------------ contractions ----- */

/* reference: cuda::gemm, src/cuda/matmul.cu:189-191 (CPU twin src/cpu/matmul.cpp:254-256).
 * Batched C[b] = A[b] . B[b]; batch dims broadcast; a transposed operand is recognised by
 * stride[-1] > stride[-2]. fp16/bf16 (and their mixes with fp32) accumulate in float32 and run
 * on the tcgen05 tensor-core path when the operands are TMA-addressable, otherwise on the SIMT
 * path; integer pairs accumulate in the output integer type. The batch counter is 64-bit
 * (the reference's wraps at 256, src/cuda/matmul.cu:45). */
tn_status tn_gemm(const tn_tensor_t* a, const tn_tensor_t* b, tn_tensor_t* dst, tn_stream_t stream);

/* matmul followed by multiplication with a scalar of dst's dtype, in one kernel:
 * dst = round(round(A.B) * scale). Replaces the gemm + scale pair of
 * `matmul(Q, K^T) * 0.125` (src/transformations.cpp:33-39 then src/operations.cpp:40-43). */
tn_status tn_gemm_scaled(const tn_tensor_t* a, const tn_tensor_t* b, const tn_scalar_t* scale,
                         tn_tensor_t* dst, tn_stream_t stream);

/* The scores-then-statistics path in one kernel: dst = matmul(a, b) [* scale] as above (scale may be
 * NULL), and for every row of dst (its last axis) the maximum, the sum and the index of the first
 * maximum, taken from the rounded result while the tensor-core epilogue still holds the row.
 * Replaces gemm + scale + three reductions that would each re-read dst
 * (src/transformations.cpp:33-39, src/operations.cpp:40-43, src/reductions.cpp:23-53). max_out and
 * sum_out have dst's dtype, argmax_out is int64; each has one element per row of dst and may be
 * NULL. Semantics are those of tn_max / tn_argsum / tn_argmax applied to dst. Results that the
 * fused epilogue does not cover (more than 256 columns, a padded row pitch, non-16-bit types) are
 * computed by the product followed by one tn_reduce_stats pass. */
tn_status tn_gemm_scaled_stats(const tn_tensor_t* a, const tn_tensor_t* b, const tn_scalar_t* scale,
                               tn_tensor_t* dst, tn_tensor_t* max_out, tn_tensor_t* sum_out,
                               tn_tensor_t* argmax_out, tn_stream_t stream);

/* reference: cuda::conv2d (two overloads), src/cuda/conv2d.cu:216-222 (CPU twin
 * src/cpu/conv2d.cpp:257-265). NCHW cross-correlation, zero padding, floor output size,
 * bias (rank 1, [Cout]) seeds the accumulator. Rank / shape mismatches return TN_ERROR. */
tn_status tn_conv2d(const tn_tensor_t* x, const tn_tensor_t* w, tn_tensor_t* y, tn_stream_t stream,
                    const size_t pad[2], const size_t stride[2]);
tn_status tn_conv2d_bias(const tn_tensor_t* x, const tn_tensor_t* w, const tn_tensor_t* bias,
                         tn_tensor_t* y, tn_stream_t stream, const size_t pad[2],
                         const size_t stride[2]);
/* Weights packed ahead of time, for callers whose convolution weights do not change between calls (no
 * reference counterpart; the reference's kernel reads NCHW weights in place, src/cuda/conv2d.cu:8-47).
 * The k x k tensor-core convolution reads its weights as [tap][Cout][Cin rounded up to 8]; tn_conv2d builds
 * that copy on every call (inside the launch that re-lays the activation). tn_conv2d_packed_weights_size
 * gives the size of the packed form (0: this dtype has none, 16-bit floats only), tn_conv2d_pack_weights
 * writes it into `packed` (device memory of that size, 16-byte aligned), and tn_conv2d_prepacked is
 * tn_conv2d / tn_conv2d_bias (bias may be null) that uses it wherever it would have packed `w` itself;
 * `w` is still passed for its shape and for the convolutions that read it in place (1 x 1, fallback). */
tn_status tn_conv2d_packed_weights_size(const tn_tensor_t* w, size_t* nbytes);
tn_status tn_conv2d_pack_weights(const tn_tensor_t* w, void* packed, tn_stream_t stream);
tn_status tn_conv2d_prepacked(const tn_tensor_t* x, const tn_tensor_t* w, const void* packed, const tn_tensor_t* bias,
                              tn_tensor_t* y, tn_stream_t stream, const size_t pad[2], const size_t stride[2]);

/* reference: cuda::conv1d, src/cuda/conv1d.cu (CPU twin src/cpu/conv1d.cpp): [N, C, L] signal,
 * [Cout, Cin, K] kernel; evaluated as the H = 1 case of conv2d. */
tn_status tn_conv1d(const tn_tensor_t* x, const tn_tensor_t* w, tn_tensor_t* y, tn_stream_t stream,
                    size_t pad, size_t stride);

/* ------------------------------------------------------------------ data movement ---- */

/* reference: cuda::outer, src/cuda/outer.cu (CPU twin src/cpu/outer.cpp:25-104): dst[i][j] =
 * a[i] * b[j] for two vectors; dtype pairs and the result type are those of the broadcast
 * multiply (the result is written as dst->dtype, never wider). */
tn_status tn_outer(const tn_tensor_t* a, const tn_tensor_t* b, tn_tensor_t* dst, tn_stream_t stream);
/* reference: cuda::repeat, src/cuda/reps.cu (CPU twin src/cpu/reps.cpp:16-97): every element along
 * `axis` repeated `reps` times in a row (repeat_interleave); dst is dense with
 * shape[axis] * reps; src may be any view of rank <= 7. */
tn_status tn_repeat(const tn_tensor_t* src, tn_tensor_t* dst, int axis, int reps, tn_stream_t stream);
/* reference: cuda::concat, src/cuda/concat.cu (CPU twin src/cpu/concat.cpp:15-127): a then b along
 * `axis` into a dense dst; operands may be any views. (The reference's CPU loop indexes the inner
 * block with the stride of dimension axis + 1 only, which is right for axis >= rank - 2; this entry
 * point concatenates correctly for every axis.) */
tn_status tn_concat(const tn_tensor_t* a, const tn_tensor_t* b, tn_tensor_t* dst, tn_stream_t stream, int axis);
/* reference: cuda::triu / cuda::tril, src/cuda/traing.cu (CPU twin src/cpu/triang.cpp:3-103):
 * matrices only; triu keeps j >= i + k, tril keeps j <= i + k, the rest becomes zero. i + k is
 * evaluated in signed arithmetic (the reference adds k to an unsigned row index, which goes wrong
 * for negative k). */
tn_status tn_triu(const tn_tensor_t* src, tn_tensor_t* dst, tn_stream_t stream, int k);
tn_status tn_tril(const tn_tensor_t* src, tn_tensor_t* dst, tn_stream_t stream, int k);
/* reference: cuda::view_as_cartesian / cuda::view_as_polar, src/cuda/complex.cu (CPU twin
 * src/cpu/complex.cpp:14-228): complex dst (interleaved re, im; dense) from two real tensors of the
 * result's rank with size-1 broadcasting: (re, im), or (rho cos theta, rho sin theta). float32 parts
 * give complex64, any float64 part complex128; polar also takes integer parts (as float32). */
tn_status tn_view_as_cartesian(const tn_tensor_t* re, const tn_tensor_t* im, tn_tensor_t* dst, tn_stream_t stream);
tn_status tn_view_as_polar(const tn_tensor_t* rho, const tn_tensor_t* theta, tn_tensor_t* dst, tn_stream_t stream);

/* ------------------------------------------------------------------ reductions ------- */

/* reference: cuda::argmax/argmin/argsum/argmean, src/cuda/argred.cu:167-213 (CPU twin
 * src/cpu/argred.cpp:289-347). Index results are int64; the first occurrence wins and NaN is
 * never selected; sum/mean keep the input dtype and accumulate in float32 (half types),
 * float64 (float32/float64) or int64 (integers), as the reference's device path does. */
tn_status tn_argmax(const tn_tensor_t* src, tn_tensor_t* dst, tn_stream_t stream, uint8_t axis);
tn_status tn_argmin(const tn_tensor_t* src, tn_tensor_t* dst, tn_stream_t stream, uint8_t axis);
tn_status tn_argsum(const tn_tensor_t* src, tn_tensor_t* dst, tn_stream_t stream, uint8_t axis);
tn_status tn_argmean(const tn_tensor_t* src, tn_tensor_t* dst, tn_stream_t stream, uint8_t axis);
/* Value maximum along an axis (= src[argmax]); the reference has no such op
 * (include/tannic/reductions.hpp:41-44 lists argmax/argmin/sum/mean only). */
tn_status tn_max(const tn_tensor_t* src, tn_tensor_t* dst, tn_stream_t stream, uint8_t axis);
/* max, sum and argmax along one axis in a single pass over src (each output may be NULL).
 * Replaces three cuda::arg* launches that would each re-read src. */
tn_status tn_reduce_stats(const tn_tensor_t* src, tn_tensor_t* max_out, tn_tensor_t* sum_out,
                          tn_tensor_t* argmax_out, tn_stream_t stream, uint8_t axis);

/* No counterpart in the reference. Sum along the last axis of a dense tensor, like tn_argsum,
 * for callers that may not allocate device memory when they call in (a server whose HBM is
 * fully budgeted at start-up; a path that cannot afford an allocator's locks and implicit
 * synchronisation). The partial sums of its two kernels live in a 192 KiB region that is part of
 * the library image on every GPU, so no cudaMalloc / cudaMallocAsync / cudaFree is ever issued.
 * Refused with TN_ERROR: a source that is not dense row-major, an axis other than the last, more
 * rows than the region has room for (one partial per row and segment: 8192 rows for float32,
 * float64 and integer sources, 12288 for float16 / bfloat16). The first call on a device resolves the region's
 * address and should be made outside stream capture. All calls on a device share the region:
 * kernels of two calls that overlap on the GPU race on it, so keep such calls ordered. */
tn_status tn_argsum_fixed_scratch(const tn_tensor_t* src, tn_tensor_t* dst, tn_stream_t stream,
                                  uint8_t axis);

/* ------------------------------------------------------------------ utilities -------- */

/* reference: cuda::cpy, src/cuda/cpy.cu:55-69 — strided -> strided copy (slice assignment). */
tn_status tn_cpy(const tn_tensor_t* src, tn_tensor_t* dst, tn_stream_t stream);
/* reference: cuda::allclose, src/cuda/val.cu:82-89 — |a-b| <= atol + rtol*|b| for all elements;
 * synchronises the stream and writes 0/1 to *close. */
tn_status tn_allclose(const tn_tensor_t* a, const tn_tensor_t* b, tn_stream_t stream, double rtol,
                      double atol, int* close);

/* reference: cuda::eq/ne/gt/ge/lt/le, which exist only as stubs that throw (src/comparisons.cpp:24-29);
 * semantics are those of the CPU twins, src/cpu/cmps.cpp:16-204: operands of one numeric dtype,
 * compared elementwise (IEEE: a NaN makes everything but != false) into a BOOLEAN result that is
 * bit-packed, element i in bit i % 8 of byte i / 8, (size + 7) / 8 bytes, unused bits zero. Operands
 * may be strided views and may broadcast extent-1 dimensions against the result. */
tn_status tn_eq(const tn_tensor_t* a, const tn_tensor_t* b, tn_tensor_t* dst, tn_stream_t stream);
tn_status tn_ne(const tn_tensor_t* a, const tn_tensor_t* b, tn_tensor_t* dst, tn_stream_t stream);
tn_status tn_gt(const tn_tensor_t* a, const tn_tensor_t* b, tn_tensor_t* dst, tn_stream_t stream);
tn_status tn_ge(const tn_tensor_t* a, const tn_tensor_t* b, tn_tensor_t* dst, tn_stream_t stream);
tn_status tn_lt(const tn_tensor_t* a, const tn_tensor_t* b, tn_tensor_t* dst, tn_stream_t stream);
tn_status tn_le(const tn_tensor_t* a, const tn_tensor_t* b, tn_tensor_t* dst, tn_stream_t stream);

/* Number of CTAs (tensor-core and staged-reduction kernels) that gave up on a bounded wait since load (0 in a
 * healthy run); synchronises the device. The reference has no device-side waits to bound. */
tn_status tn_device_errors(unsigned int* count);

/* The product, written into `dst` and, tile by tile from the same kernel, into up to seven further buffers of the
 * same dtype, shape and strides: memory of OTHER GPUs mapped into this process (symmetric memory, IPC). The epilogue
 * stores every 16 bytes of a result tile into each of them with plain stores that NVLink carries while the tensor
 * cores work on the next tile, so a batch-sharded GEMM whose whole result every GPU needs is one kernel, not a GEMM
 * followed by an all-gather. The caller orders the exchange (nobody reads a mirror before the kernel and a fence
 * over the group have completed; `tannic_b200.shard.matmul_into_all` does it with two one-element all-reduces).
 * 16-bit operands and result on the tensor-core path with 16-byte aligned bases and pitches; otherwise
 * TN_ERROR (dst alone is then written). No reference counterpart. */
tn_status tn_gemm_mirrored(const tn_tensor_t* a, const tn_tensor_t* b, tn_tensor_t* dst, const tn_tensor_t* const* mirrors,
                           int n_mirrors, tn_stream_t stream);

/* The tensor-core GEMM and convolution kernels are persistent, one thread block per SM, and a block fills
 * its SM's shared memory: while one runs, no kernel of another stream gets an SM. A caller that wants a
 * communication kernel (an NCCL send/receive of the rows just produced) to run UNDER the next GEMM sets a
 * margin: these kernels then launch on (SM count - margin) SMs. Process-wide, 0..64, default 0. No reference
 * counterpart. */
tn_status tn_set_sm_margin(int sms);

/* Diagnostics, no reference counterpart: launches of the tensor-core GEMM since load, by variant:
 * [0] general kernel, [1] packed-row epilogue, [2] packed rows + fused row statistics, [3] stationary A
 * (short K, A held in tensor memory). Convolutions through the implicit GEMM count under [0]. */
tn_status tn_gemm_path_launches(uint64_t counts[4]);

/* Failure-detection self-test, no reference counterpart: launches one warp that waits, with the same
 * bounded wait the tensor-core kernels use, on a barrier nothing ever completes. The wait runs out
 * after `polls` polls (about 64 ns each, capped at the kernels' own limit), the kernel returns
 * normally and the abort counter rises by one, so tn_device_errors() and the next synchronising
 * call report it. Nothing faults or hangs. */
tn_status tn_selftest_bounded_wait(const tn_device_t* device, tn_stream_t stream, unsigned int polls);

/* Number of kernels this library has launched on the calling process since load (all threads).
 * Used by the benchmark to count launches inside its timed region. */
uint64_t tn_launch_count(void);

#ifdef __cplusplus
}
#endif

#endif /* TANNIC_B200_H */
