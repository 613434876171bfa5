"""Host-side mirror of Tannic's operator front-end for the device path, over torch CUDA tensors.

The reference's front-end is header-only C++ (expression templates); what it decides before a
kernel runs is small and is restated here so that tests and the benchmark read like the
reference's own: result dtype (`max` of the enum order for elementwise ops,
include/tannic/operations.hpp:133-135; the matmul table, include/tannic/transformations.hpp:87-152;
int64 for argmax/argmin, include/tannic/reductions.hpp:101-119), NumPy broadcast shape
(operations.hpp:137-152), matmul batch broadcast (transformations.hpp:161-202), conv output
shape (convolutions.hpp:88-109), axis normalisation / keepdim (reductions.hpp:101-193). The
result is allocated dense and the C ABI entry point is called on the tensors' own memory.
torch supplies device memory only; no torch kernel computes anything here.
"""
from __future__ import annotations

import builtins as _b
import ctypes as C
from typing import Sequence

import torch

from . import _abi as A

TORCH_TO_TN = {
    torch.int8: A.INT8, torch.int16: A.INT16, torch.int32: A.INT32, torch.int64: A.INT64,
    torch.float16: A.FLOAT16, torch.bfloat16: A.BFLOAT16, torch.float32: A.FLOAT32, torch.float64: A.FLOAT64,
    torch.complex64: A.COMPLEX64, torch.complex128: A.COMPLEX128,
}
TN_TO_TORCH = {v: k for k, v in TORCH_TO_TN.items()}


def desc(t: torch.Tensor) -> A.TensorT:
    """tn_tensor_t over a torch tensor's storage (CUDA -> DEVICE environment, CPU -> HOST)."""
    if t.dtype not in TORCH_TO_TN:
        raise A.TannicError(A.UNSUPPORTED_DTYPE, f"torch dtype {t.dtype} has no Tannic equivalent")
    device = t.device.index if t.is_cuda else None
    if t.is_cuda and device is None:
        device = torch.cuda.current_device()
    return A.make_tensor(t.data_ptr(), tuple(t.shape), tuple(t.stride()), TORCH_TO_TN[t.dtype], device,
                         pinned=(not t.is_cuda) and t.is_pinned())


def current_stream(t: torch.Tensor) -> A.StreamT:
    return A.StreamT(torch.cuda.current_stream(t.device).cuda_stream)


def _empty(shape, tn_dtype, like: torch.Tensor) -> torch.Tensor:
    return torch.empty(tuple(shape), dtype=TN_TO_TORCH[tn_dtype], device=like.device)


def broadcast_shape(a: Sequence[int], b: Sequence[int]) -> tuple:
    """include/tannic/operations.hpp:137-152"""
    rank = _b.max(len(a), len(b))
    out = []
    for i in range(rank):
        x = a[len(a) - rank + i] if i >= rank - len(a) else 1
        y = b[len(b) - rank + i] if i >= rank - len(b) else 1
        if x != y and x != 1 and y != 1:
            raise ValueError("Shapes are not broadcast-compatible.")
        out.append(_b.max(x, y))
    return tuple(out)


def _binary(name: str, a: torch.Tensor, b: torch.Tensor, out_dtype: int | None = None) -> torch.Tensor:
    dt = out_dtype if out_dtype is not None else _b.max(TORCH_TO_TN[a.dtype], TORCH_TO_TN[b.dtype])
    out = _empty(broadcast_shape(a.shape, b.shape), dt, a)
    da, db, dd = desc(a), desc(b), desc(out)
    A.check(getattr(A.lib(), f"tn_{name}")(C.byref(da), C.byref(db), C.byref(dd), current_stream(a)))
    return out


def add(a, b, **kw): return _binary("add", a, b, **kw)
def sub(a, b, **kw): return _binary("sub", a, b, **kw)
def mul(a, b, **kw): return _binary("mul", a, b, **kw)
def pow(a, b, **kw): return _binary("pow", a, b, **kw)  # noqa: A001


def _compare(name: str, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """include/tannic/comparisons.hpp:40-130: boolean result of the operands' shape, bit-packed
    (element i in bit i % 8 of byte i / 8). Returned as the packed uint8 buffer of (n + 7) // 8 bytes
    together with the logical shape via `unpack_bits`."""
    if a.dtype != b.dtype:
        raise A.TannicError(A.UNSUPPORTED_DTYPE, "comparison operands must share a dtype")
    shape = broadcast_shape(a.shape, b.shape)
    rank = len(shape)
    a = a.reshape((1,) * (rank - a.dim()) + tuple(a.shape))
    b = b.reshape((1,) * (rank - b.dim()) + tuple(b.shape))
    n = 1
    for s in shape:
        n *= s
    packed = torch.empty(((n + 7) // 8,), dtype=torch.uint8, device=a.device)
    dense, run = [], 1
    for extent in reversed(shape):
        dense.insert(0, run)
        run *= extent
    dd = A.make_tensor(packed.data_ptr(), shape, dense, A.BOOLEAN,
                       a.device.index if a.device.index is not None else torch.cuda.current_device())
    da, db = desc(a), desc(b)
    A.check(getattr(A.lib(), f"tn_{name}")(C.byref(da), C.byref(db), C.byref(dd), current_stream(a)))
    return packed


def unpack_bits(packed: torch.Tensor, shape) -> torch.Tensor:
    """Bit-packed boolean buffer -> torch.bool tensor of `shape` (host side)."""
    n = 1
    for s in shape:
        n *= s
    bytes_ = packed.cpu().to(torch.int32)
    bits = (bytes_.unsqueeze(-1) >> torch.arange(8, dtype=torch.int32)) & 1
    return bits.reshape(-1)[:n].to(torch.bool).reshape(tuple(shape))


def eq(a, b): return _compare("eq", a, b)
def ne(a, b): return _compare("ne", a, b)
def gt(a, b): return _compare("gt", a, b)
def ge(a, b): return _compare("ge", a, b)
def lt(a, b): return _compare("lt", a, b)
def le(a, b): return _compare("le", a, b)


def _unary(name: str, x: torch.Tensor, *extra) -> torch.Tensor:
    out = _empty(x.shape, TORCH_TO_TN[x.dtype], x)
    dx, dd = desc(x), desc(out)
    A.check(getattr(A.lib(), f"tn_{name}")(C.byref(dx), C.byref(dd), current_stream(x), *extra))
    return out


def neg(x): return _unary("neg", x)
def repack(x): return _unary("repack", x)
def log(x): return _unary("log", x)
def exp(x): return _unary("exp", x)
def sqrt(x): return _unary("sqrt", x)
def rsqrt(x, eps: float = 0.0): return _unary("rsqrt", x, C.c_float(eps))
def abs(x): return _unary("abs", x)  # noqa: A001
def sin(x): return _unary("sin", x)
def cos(x): return _unary("cos", x)
def tan(x): return _unary("tan", x)
def sinh(x): return _unary("sinh", x)
def cosh(x): return _unary("cosh", x)
def tanh(x): return _unary("tanh", x)


def _scalar(value, tn_dtype: int):
    """A host scalar cast to the tensor's dtype first, as `tensor * 0.125` does in the reference
    (include/tannic/operations.hpp:295-313, include/tannic/scalars.hpp:36-52)."""
    holder = torch.tensor([value], dtype=TN_TO_TORCH[tn_dtype])
    return holder, A.ScalarT(holder.data_ptr(), tn_dtype)


def scale(x: torch.Tensor, value) -> torch.Tensor:
    out = _empty(x.shape, TORCH_TO_TN[x.dtype], x)
    holder, sc = _scalar(value, TORCH_TO_TN[x.dtype])
    dx, dd = desc(x), desc(out)
    A.check(A.lib().tn_scale(C.byref(dx), C.byref(sc), C.byref(dd), current_stream(x)))
    return out


def program(inputs: Sequence[torch.Tensor], nodes: Sequence[tuple], out: torch.Tensor | None = None) -> torch.Tensor:
    """Fused elementwise program. `nodes` are (opcode, lhs, rhs[, imm]) with value ids 0..3 for the
    inputs and 4+k for node k. `out` (optional) is a preallocated result of the broadcast shape."""
    shape = tuple(inputs[0].shape)
    for t in inputs[1:]:
        shape = broadcast_shape(shape, t.shape)
    if out is None:
        out = _empty(shape, TORCH_TO_TN[inputs[0].dtype], inputs[0])
    elif tuple(out.shape) != shape or out.dtype != inputs[0].dtype:
        raise ValueError("out must have the broadcast shape and the inputs' dtype")
    descs = [desc(t) for t in inputs]
    ptrs = (C.POINTER(A.TensorT) * len(descs))(*[C.pointer(d) for d in descs])
    arr = (A.EltwiseNode * len(nodes))()
    for k, nd in enumerate(nodes):
        arr[k].opcode, arr[k].lhs, arr[k].rhs = nd[0], nd[1], nd[2]
        arr[k].imm = nd[3] if len(nd) > 3 else 0.0
    dd = desc(out)
    A.check(A.lib().tn_eltwise_program(ptrs, len(descs), arr, len(nodes), C.byref(dd), current_stream(out)))
    return out


def program_host(inputs: Sequence[torch.Tensor], nodes: Sequence[tuple], out_host: torch.Tensor, device: int = 0, chunks: int = 0) -> torch.Tensor:
    """Fused elementwise program over HOST tensors through tn_eltwise_program_host: chunked copy-in,
    kernel and copy-out overlapped on three streams inside the library; returns when `out_host` is
    complete. Host tensors should be pinned (see pinned_empty), otherwise the copies are synchronous."""
    descs = [desc(t) for t in inputs]
    ptrs = (C.POINTER(A.TensorT) * len(descs))(*[C.pointer(d) for d in descs])
    arr = (A.EltwiseNode * len(nodes))()
    for k, nd in enumerate(nodes):
        arr[k].opcode, arr[k].lhs, arr[k].rhs = nd[0], nd[1], nd[2]
        arr[k].imm = nd[3] if len(nd) > 3 else 0.0
    dd = desc(out_host)
    dev = A.DeviceT(device)
    A.check(A.lib().tn_eltwise_program_host(C.byref(dev), ptrs, len(descs), arr, len(nodes), C.byref(dd), chunks))
    return out_host


class PinnedBuffer:
    """Pinned host memory from the backend's allocator, preferably on the memory node of `device`
    (tn_host_allocate_pinned_near), viewed as a torch tensor. Freed when the object is collected."""

    def __init__(self, shape, dtype: torch.dtype, device: int = 0):
        self.nbytes = int(torch.empty((), dtype=dtype).element_size())
        for n in shape:
            self.nbytes *= int(n)
        self.address = C.c_void_p()
        dev = A.DeviceT(device)
        A.check(A.lib().tn_host_allocate_pinned_near(C.byref(dev), _b.max(self.nbytes, 1), C.byref(self.address)))
        raw = (C.c_uint8 * _b.max(self.nbytes, 1)).from_address(self.address.value)
        self.tensor = torch.frombuffer(raw, dtype=torch.uint8, count=self.nbytes).view(dtype).reshape(tuple(shape))

    def __del__(self):
        if getattr(self, "address", None) is not None and self.address.value:
            try:
                A.lib().tn_host_free_pinned(self.address)
            except Exception:
                pass
            self.address = None


def numa_node(device: int = 0) -> int:
    node = C.c_int(-1)
    dev = A.DeviceT(device)
    A.check(A.lib().tn_device_numa_node(C.byref(dev), C.byref(node)))
    return node.value


def bind_thread_near(device: int = 0) -> int:
    node = C.c_int(-1)
    dev = A.DeviceT(device)
    A.check(A.lib().tn_bind_thread_near(C.byref(dev), C.byref(node)))
    return node.value


def _matmul_dtype(a: int, b: int) -> int:
    """include/tannic/transformations.hpp:87-152"""
    ints = (A.INT8, A.INT16, A.INT32, A.INT64)
    if a in ints and b in ints:
        if A.INT64 in (a, b) or (a == A.INT32 and b == A.INT32):
            return A.INT64
        return A.INT32
    halves = (A.FLOAT16, A.BFLOAT16)
    for h, o in ((a, b), (b, a)):
        if h in halves:
            if o == h:
                return h
            if o in halves:
                return A.FLOAT16
            if o in (A.INT8, A.INT16):
                return h
            if o == A.INT32 or o == A.FLOAT32:
                return A.FLOAT32
            if o == A.INT64 or o == A.FLOAT64:
                return A.FLOAT64
    if A.FLOAT64 in (a, b):
        return A.FLOAT64
    if A.FLOAT32 in (a, b) and (a in (A.FLOAT32, A.INT32)) and (b in (A.FLOAT32, A.INT32)):
        return A.FLOAT32
    raise A.TannicError(A.UNSUPPORTED_DTYPE, "Unsuported dtypes")


def matmul(a: torch.Tensor, b: torch.Tensor, scale_by=None, out_dtype: int | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """matmul(a, b) [* scalar]; transposed operands arrive as strided views (`b.transpose(-1, -2)`).
    `out` (optional) is a preallocated result of the right shape and dtype, as the reference's
    Callback hands one to the kernel."""
    if a.dim() < 2 or b.dim() < 2:
        raise ValueError("Inputs must have rank >= 2")
    if a.shape[-1] != b.shape[-2]:
        raise ValueError("Inner dimensions must match for matmul")
    batch = broadcast_shape(a.shape[:-2], b.shape[:-2])
    dt = out_dtype if out_dtype is not None else _matmul_dtype(TORCH_TO_TN[a.dtype], TORCH_TO_TN[b.dtype])
    if out is None:
        out = _empty(batch + (a.shape[-2], b.shape[-1]), dt, a)
    elif tuple(out.shape) != batch + (a.shape[-2], b.shape[-1]) or out.dtype != TN_TO_TORCH[dt]:
        raise ValueError("out must have the result's shape and dtype")
    da, db, dd = desc(a), desc(b), desc(out)
    if scale_by is None:
        A.check(A.lib().tn_gemm(C.byref(da), C.byref(db), C.byref(dd), current_stream(a)))
    else:
        holder, sc = _scalar(scale_by, dt)
        A.check(A.lib().tn_gemm_scaled(C.byref(da), C.byref(db), C.byref(sc), C.byref(dd), current_stream(a)))
    return out


def matmul_mirrored(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, mirrors) -> torch.Tensor:
    """matmul(a, b) into `out` and, from the same kernel, into every tensor of `mirrors` (views of other GPUs'
    memory with out's shape, dtype and strides): tn_gemm_mirrored."""
    da, db, dd = desc(a), desc(b), desc(out)
    records = [desc(m) for m in mirrors]
    ptrs = (C.POINTER(A.TensorT) * _b.max(1, len(records)))(*[C.pointer(r) for r in records])
    A.check(A.lib().tn_gemm_mirrored(C.byref(da), C.byref(db), C.byref(dd), ptrs, len(records), current_stream(a)))
    return out


def matmul_stats(a: torch.Tensor, b: torch.Tensor, scale_by=None, out: torch.Tensor | None = None):
    """(S, max, sum, argmax) with S = matmul(a, b) [* scalar] and the three statistics taken along S's
    last axis in the same kernel where the shape allows (tn_gemm_scaled_stats)."""
    batch = broadcast_shape(a.shape[:-2], b.shape[:-2])
    dt = _matmul_dtype(TORCH_TO_TN[a.dtype], TORCH_TO_TN[b.dtype])
    shape = batch + (a.shape[-2], b.shape[-1])
    if out is None:
        out = _empty(shape, dt, a)
    mx, sm, am = _empty(shape[:-1], dt, a), _empty(shape[:-1], dt, a), _empty(shape[:-1], A.INT64, a)
    da, db, dd, dmx, dsm, dam = desc(a), desc(b), desc(out), desc(mx), desc(sm), desc(am)
    sc = None
    if scale_by is not None:
        holder, sc = _scalar(scale_by, dt)
    A.check(A.lib().tn_gemm_scaled_stats(C.byref(da), C.byref(db), C.byref(sc) if sc is not None else None, C.byref(dd),
                                         C.byref(dmx), C.byref(dsm), C.byref(dam), current_stream(a)))
    return out, mx, sm, am


def _pair(v):
    return (v, v) if isinstance(v, int) else tuple(v)


def pack_conv_weights(w: torch.Tensor) -> torch.Tensor | None:
    """The weights in the layout the k x k tensor-core convolution reads (tn_conv2d_pack_weights), for
    `convolve2D(..., packed=...)`; None for dtypes that have no packed form."""
    n = C.c_size_t(0)
    dw = desc(w)
    A.check(A.lib().tn_conv2d_packed_weights_size(C.byref(dw), C.byref(n)))
    if n.value == 0:
        return None
    packed = torch.empty(n.value // 2, dtype=torch.int16, device=w.device)
    A.check(A.lib().tn_conv2d_pack_weights(C.byref(dw), C.c_void_p(packed.data_ptr()), current_stream(w)))
    return packed


def convolve2D(x: torch.Tensor, w: torch.Tensor, stride=1, padding=0, bias: torch.Tensor | None = None,
               packed: torch.Tensor | None = None) -> torch.Tensor:
    """include/tannic/convolutions.hpp:185-273; note the reference's argument order (stride, padding).
    `packed`: the result of pack_conv_weights(w), for weights that do not change between calls."""
    if x.dim() != 4 or w.dim() != 4:
        raise ValueError("Only rank 4 tensors supported.")
    if x.dtype != w.dtype or (bias is not None and bias.dtype != x.dtype):
        raise ValueError("Dtypes must match in convolutions.")
    if x.shape[1] != w.shape[1]:
        raise ValueError("Input channels must match kernel channels.")
    s, p = _pair(stride), _pair(padding)
    ho = (x.shape[2] + 2 * p[0] - w.shape[2]) // s[0] + 1
    wo = (x.shape[3] + 2 * p[1] - w.shape[3]) // s[1] + 1
    out = _empty((x.shape[0], w.shape[0], ho, wo), TORCH_TO_TN[x.dtype], x)
    pad = (C.c_size_t * 2)(*p)
    strd = (C.c_size_t * 2)(*s)
    dx, dw, dd = desc(x), desc(w), desc(out)
    if packed is not None:
        dbias = desc(bias) if bias is not None else None
        A.check(A.lib().tn_conv2d_prepacked(C.byref(dx), C.byref(dw), C.c_void_p(packed.data_ptr()), C.byref(dbias) if dbias is not None else None,
                                            C.byref(dd), current_stream(x), pad, strd))
    elif bias is None:
        A.check(A.lib().tn_conv2d(C.byref(dx), C.byref(dw), C.byref(dd), current_stream(x), pad, strd))
    else:
        dbias = desc(bias)
        A.check(A.lib().tn_conv2d_bias(C.byref(dx), C.byref(dw), C.byref(dbias), C.byref(dd), current_stream(x), pad, strd))
    return out


def convolve1D(x: torch.Tensor, w: torch.Tensor, stride: int = 1, padding: int = 0) -> torch.Tensor:
    """include/tannic/convolutions.hpp (Convolution<1>): [N, C, L] signal, [Cout, Cin, K] kernel."""
    if x.dim() != 3 or w.dim() != 3:
        raise ValueError("Only rank 3 tensors supported.")
    if x.dtype != w.dtype:
        raise ValueError("Dtypes must match in convolutions.")
    if x.shape[1] != w.shape[1]:
        raise ValueError("Input channels must match kernel channels.")
    lo = (x.shape[2] + 2 * padding - w.shape[2]) // stride + 1
    out = _empty((x.shape[0], w.shape[0], lo), TORCH_TO_TN[x.dtype], x)
    dx, dw, dd = desc(x), desc(w), desc(out)
    A.check(A.lib().tn_conv1d(C.byref(dx), C.byref(dw), C.byref(dd), current_stream(x), padding, stride))
    return out


def outer(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """include/tannic/transformations.hpp (Outer): two vectors, promoted dtype, shape [len(a), len(b)]."""
    if a.dim() != 1 or b.dim() != 1:
        raise ValueError("Outer product of tensors with rank more than 1 not supported.")
    out = _empty((a.shape[0], b.shape[0]), _b.max(TORCH_TO_TN[a.dtype], TORCH_TO_TN[b.dtype]), a)
    da, db, dd = desc(a), desc(b), desc(out)
    A.check(A.lib().tn_outer(C.byref(da), C.byref(db), C.byref(dd), current_stream(a)))
    return out


def repeat(x: torch.Tensor, repeats: int, axis: int) -> torch.Tensor:
    """include/tannic/transformations.hpp (Repetition): every element along `axis` `repeats` times in a row."""
    axis = axis % x.dim()
    shape = list(x.shape)
    shape[axis] *= repeats
    out = _empty(shape, TORCH_TO_TN[x.dtype], x)
    dx, dd = desc(x), desc(out)
    A.check(A.lib().tn_repeat(C.byref(dx), C.byref(dd), axis, repeats, current_stream(x)))
    return out


def concatenate(a: torch.Tensor, b: torch.Tensor, axis: int = 0) -> torch.Tensor:
    """include/tannic/transformations.hpp (Concatenation): same dtype, same shape off the axis."""
    if a.dtype != b.dtype:
        raise ValueError("Cannot concatenate tensors of different dtypes.")
    axis = axis % a.dim()
    shape = list(a.shape)
    shape[axis] += b.shape[axis]
    out = _empty(shape, TORCH_TO_TN[a.dtype], a)
    da, db, dd = desc(a), desc(b), desc(out)
    A.check(A.lib().tn_concat(C.byref(da), C.byref(db), C.byref(dd), current_stream(a), axis))
    return out


def _triangular(name: str, x: torch.Tensor, k: int) -> torch.Tensor:
    out = _empty(x.shape, TORCH_TO_TN[x.dtype], x)
    dx, dd = desc(x), desc(out)
    A.check(getattr(A.lib(), f"tn_{name}")(C.byref(dx), C.byref(dd), current_stream(x), k))
    return out


def triu(x, k: int = 0): return _triangular("triu", x, k)
def tril(x, k: int = 0): return _triangular("tril", x, k)


def _complex_from(name: str, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """include/tannic/complex.hpp (Cartesian / Polar): complex64 from float32 parts, complex128 as soon
    as one part is float64."""
    wide = torch.float64 in (a.dtype, b.dtype)
    out = _empty(broadcast_shape(a.shape, b.shape), A.COMPLEX128 if wide else A.COMPLEX64, a)
    rank = out.dim()
    a = a.reshape((1,) * (rank - a.dim()) + tuple(a.shape))
    b = b.reshape((1,) * (rank - b.dim()) + tuple(b.shape))
    da, db, dd = desc(a), desc(b), desc(out)
    A.check(getattr(A.lib(), f"tn_{name}")(C.byref(da), C.byref(db), C.byref(dd), current_stream(a)))
    return out


def cartesian(re, im): return _complex_from("view_as_cartesian", re, im)
def polar(rho, theta): return _complex_from("view_as_polar", rho, theta)


def _reduced_shape(shape, axis: int, keepdim: bool):
    shape = list(shape)
    if keepdim:
        shape[axis] = 1
    else:
        del shape[axis]
    return tuple(shape)


def _reduce(name: str, x: torch.Tensor, axis: int, keepdim: bool, out_dtype: int) -> torch.Tensor:
    if x.dim() == 0:
        raise ValueError("cannot reduce a rank-0 tensor")
    ax = axis + x.dim() if axis < 0 else axis
    out = _empty(_reduced_shape(x.shape, ax, keepdim), out_dtype, x)
    dx, dd = desc(x), desc(out)
    A.check(getattr(A.lib(), f"tn_{name}")(C.byref(dx), C.byref(dd), current_stream(x), C.c_uint8(ax)))
    return out


def argmax(x, axis=-1, keepdim=False): return _reduce("argmax", x, axis, keepdim, A.INT64)
def argmin(x, axis=-1, keepdim=False): return _reduce("argmin", x, axis, keepdim, A.INT64)
def sum(x, axis=-1, keepdim=False): return _reduce("argsum", x, axis, keepdim, TORCH_TO_TN[x.dtype])  # noqa: A001
def mean(x, axis=-1, keepdim=False): return _reduce("argmean", x, axis, keepdim, TORCH_TO_TN[x.dtype])
def max(x, axis=-1, keepdim=False): return _reduce("max", x, axis, keepdim, TORCH_TO_TN[x.dtype])  # noqa: A001


def reduce_stats(x: torch.Tensor, axis=-1, keepdim=False):
    """(max, sum, argmax) along `axis` from one pass over x."""
    ax = axis + x.dim() if axis < 0 else axis
    shape = _reduced_shape(x.shape, ax, keepdim)
    mx = _empty(shape, TORCH_TO_TN[x.dtype], x)
    sm = _empty(shape, TORCH_TO_TN[x.dtype], x)
    am = _empty(shape, A.INT64, x)
    dx, dmx, dsm, dam = desc(x), desc(mx), desc(sm), desc(am)
    A.check(A.lib().tn_reduce_stats(C.byref(dx), C.byref(dmx), C.byref(dsm), C.byref(dam), current_stream(x), C.c_uint8(ax)))
    return mx, sm, am


def allclose(a: torch.Tensor, b: torch.Tensor, rtol: float = 1e-5, atol: float = 1e-8) -> bool:
    """include/tannic/comparisons.hpp:128 defaults."""
    da, db = desc(a), desc(b)
    flag = C.c_int(0)
    A.check(A.lib().tn_allclose(C.byref(da), C.byref(db), current_stream(a), rtol, atol, C.byref(flag)))
    return bool(flag.value)


def cpy(src: torch.Tensor, dst: torch.Tensor) -> None:
    ds, dd = desc(src), desc(dst)
    A.check(A.lib().tn_cpy(C.byref(ds), C.byref(dd), current_stream(dst)))


def device_errors() -> int:
    n = C.c_uint(0)
    A.check(A.lib().tn_device_errors(C.byref(n)))
    return n.value


def program_jit(mode: int) -> None:
    """0: never compile programs at run time, 1: for results of 2^20 elements and more, 2: always."""
    A.check(A.lib().tn_program_jit_enable(int(mode)))


def program_jit_stats() -> dict:
    """Run-time compiled programs so far, failed compilations, and whether NVRTC is usable."""
    c, f, a, d = C.c_uint(0), C.c_uint(0), C.c_uint(0), C.c_uint(0)
    A.check(A.lib().tn_program_jit_stats(C.byref(c), C.byref(f), C.byref(a), C.byref(d)))
    return {"compiled": c.value, "failed": f.value, "available": bool(a.value), "from_disk": d.value, "log": (A.lib().tn_program_jit_log() or b"").decode(errors="replace")}


def sm_margin(sms: int) -> None:
    """SMs the persistent tensor-core kernels leave free for kernels of other streams (0 = none)."""
    A.check(A.lib().tn_set_sm_margin(int(sms)))


def gemm_path_launches() -> dict:
    """Tensor-core GEMM launches since load, by kernel variant."""
    c = (C.c_uint64 * 4)()
    A.check(A.lib().tn_gemm_path_launches(c))
    return {"general": c[0], "packed": c[1], "packed_stats": c[2], "stationary": c[3]}


def launch_count() -> int:
    return int(A.lib().tn_launch_count())
