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


class HostPipeline:
    """Host buffers in, host buffer out, for a fused elementwise program: the rows are cut into chunks and
    the host-to-device copy of chunk c + 1, the kernel of chunk c and the device-to-host copy of chunk
    c - 1 run at the same time on three streams (PCIe is full duplex), so a call costs about one
    direction's transfer time instead of both plus the kernel. Inputs whose leading extent equals the
    result's are chunked; smaller (broadcast) inputs are copied whole first. Host tensors should be
    pinned, otherwise the copies are synchronous. Device staging memory is kept between calls.

    The reference moves data with one synchronous cudaMemcpy per call (src/cuda/mem.cu:54-90) and has no
    pinned host allocator (src/resources.cpp:24-38 throws)."""

    def __init__(self, device: int | torch.device | None = None, chunks: int = 8):
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.chunks = chunks
        self.s_in, self.s_run, self.s_out = (torch.cuda.Stream(self.device) for _ in range(3))
        self._staging: dict = {}

    def _dev(self, key, shape, dtype):
        buf = self._staging.get(key)
        if buf is None or tuple(buf.shape) != tuple(shape) or buf.dtype != dtype:
            buf = torch.empty(tuple(shape), dtype=dtype, device=self.device)
            self._staging[key] = buf
        return buf

    def program(self, inputs: Sequence[torch.Tensor], nodes: Sequence[tuple], out_host: torch.Tensor) -> torch.Tensor:
        shape = tuple(inputs[0].shape)
        for t in inputs[1:]:
            shape = broadcast_shape(shape, t.shape)
        if tuple(out_host.shape) != shape:
            raise ValueError("out_host must have the broadcast shape")
        rows = shape[0] if len(shape) > 1 else 1
        chunked = [len(shape) > 1 and t.dim() == len(shape) and t.shape[0] == rows and rows > 1 for t in inputs]
        dev_in = [self._dev(("in", k), t.shape, t.dtype) for k, t in enumerate(inputs)]
        dev_out = self._dev(("out",), shape, out_host.dtype)
        caller = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_run, self.s_out):
            s.wait_stream(caller)
        with torch.cuda.stream(self.s_in):
            for k, t in enumerate(inputs):
                if not chunked[k]:
                    dev_in[k].copy_(t, non_blocking=True)
        n = _b.max(1, _b.min(self.chunks, rows)) if any(chunked) else 1
        bounds = [(rows * c) // n for c in range(n + 1)]
        for c in range(n):
            lo, hi = bounds[c], bounds[c + 1]
            if hi == lo:
                continue
            with torch.cuda.stream(self.s_in):
                for k, t in enumerate(inputs):
                    if chunked[k]:
                        dev_in[k][lo:hi].copy_(t[lo:hi], non_blocking=True)
                arrived = self.s_in.record_event()
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(arrived)
                views = [dev_in[k][lo:hi] if chunked[k] else dev_in[k] for k in range(len(inputs))]
                program(views, nodes, out=dev_out[lo:hi] if any(chunked) else dev_out)
                done = self.s_run.record_event()
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(done)
                (out_host[lo:hi] if any(chunked) else out_host).copy_(dev_out[lo:hi] if any(chunked) else dev_out, non_blocking=True)
        caller.wait_stream(self.s_out)
        return out_host


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


def matmul(a: torch.Tensor, b: torch.Tensor, scale_by=None, out_dtype: int | None = None) -> torch.Tensor:
    """matmul(a, b) [* scalar]; transposed operands arrive as strided views (`b.transpose(-1, -2)`)."""
    if a.dim() < 2 or b.dim() < 2:
        raise ValueError("Inputs must have rank >= 2")
    if a.shape[-1] != b.shape[-2]:
        raise ValueError("Inner dimensions must match for matmul")
    batch = broadcast_shape(a.shape[:-2], b.shape[:-2])
    dt = out_dtype if out_dtype is not None else _matmul_dtype(TORCH_TO_TN[a.dtype], TORCH_TO_TN[b.dtype])
    out = _empty(batch + (a.shape[-2], b.shape[-1]), dt, a)
    da, db, dd = desc(a), desc(b), desc(out)
    if scale_by is None:
        A.check(A.lib().tn_gemm(C.byref(da), C.byref(db), C.byref(dd), current_stream(a)))
    else:
        holder, sc = _scalar(scale_by, dt)
        A.check(A.lib().tn_gemm_scaled(C.byref(da), C.byref(db), C.byref(sc), C.byref(dd), current_stream(a)))
    return out


def _pair(v):
    return (v, v) if isinstance(v, int) else tuple(v)


def convolve2D(x: torch.Tensor, w: torch.Tensor, stride=1, padding=0, bias: torch.Tensor | None = None) -> torch.Tensor:
    """include/tannic/convolutions.hpp:185-273; note the reference's argument order (stride, padding)."""
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
    if bias is None:
        A.check(A.lib().tn_conv2d(C.byref(dx), C.byref(dw), C.byref(dd), current_stream(x), pad, strd))
    else:
        dbias = desc(bias)
        A.check(A.lib().tn_conv2d_bias(C.byref(dx), C.byref(dw), C.byref(dbias), C.byref(dd), current_stream(x), pad, strd))
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


def launch_count() -> int:
    return int(A.lib().tn_launch_count())
