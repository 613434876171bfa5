"""TEST INFRASTRUCTURE — Python handles on the parity oracle.

`oracle.port()`  loads oracle/liboracle.so, the C restatement of the reference's algorithms
                 (tannic_oracle.c);
`oracle.ref()`   loads oracle/_ref/libtannic_ref.so, the reference's own CPU kernels compiled
                 from its sources (None when it was never built on this machine).

Only tests/, `__graft_entry__.smoke()` and the CPU-baseline leg of bench.py may import this
package; the product (tannic_b200) never does, and this package imports nothing from the product:
its records and front-end rules are its own (`_records.py`).
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import torch

from . import _records as A

HERE = Path(__file__).resolve().parent
PORT_PATH = HERE / "liboracle.so"
REF_PATH = HERE / "_ref" / "libtannic_ref.so"

ACC_STORAGE, ACC_WIDE = 0, 1
BINARY = {"add": 0, "sub": 1, "mul": 2, "pow": 3}
UNARY = {"neg": 0, "repack": 1, "log": 2, "exp": 3, "sqrt": 4, "rsqrt": 5, "abs": 6, "sin": 7, "cos": 8, "tan": 9,
         "sinh": 10, "cosh": 11, "tanh": 12}
REDUCE = {"argmax": 0, "argmin": 1, "sum": 2, "mean": 3, "max": 4}
COMPARE = {"eq": 0, "ne": 1, "gt": 2, "ge": 3, "lt": 4, "le": 5}

_TP = C.POINTER(A.TensorT)
_port = None
_ref = None


def build(with_reference: bool = True, reference: str | None = None) -> None:
    """Compile the C restatement and, when `reference` (or $TANNIC_REFERENCE) names the reference's
    source tree, its CPU kernels into oracle/_ref."""
    import os
    reference = reference or os.environ.get("TANNIC_REFERENCE", "")
    target = "all" if with_reference and reference else str(PORT_PATH)
    subprocess.run(["make", "-s", "-C", str(HERE), target, f"REFERENCE={reference}"], check=True)


def port() -> C.CDLL:
    global _port
    if _port is None:
        if not PORT_PATH.exists():
            build(with_reference=False)
        lib = C.CDLL(str(PORT_PATH))
        lib.orc_binary.argtypes = [C.c_int, _TP, _TP, _TP]
        lib.orc_unary.argtypes = [C.c_int, _TP, _TP, C.c_float]
        lib.orc_scale.argtypes = [_TP, C.POINTER(A.ScalarT), _TP]
        lib.orc_gemm.argtypes = [_TP, _TP, _TP, C.c_int, C.c_int]
        lib.orc_conv2d.argtypes = [_TP, _TP, _TP, _TP, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t), C.c_int]
        lib.orc_reduce.argtypes = [C.c_int, _TP, _TP, C.c_uint8, C.c_int]
        lib.orc_cpy.argtypes = [_TP, _TP]
        lib.orc_allclose.argtypes = [_TP, _TP, C.c_double, C.c_double, C.POINTER(C.c_int)]
        lib.orc_compare.argtypes = [C.c_int, _TP, _TP, _TP]
        lib.orc_repeat.argtypes = [_TP, _TP, C.c_int, C.c_int]
        lib.orc_concat.argtypes = [_TP, _TP, _TP, C.c_int]
        lib.orc_triangular.argtypes = [_TP, _TP, C.c_int, C.c_int]
        lib.orc_complex_pair.argtypes = [_TP, _TP, _TP, C.c_int]
        lib.orc_fill.argtypes = [C.c_void_p, C.c_int, C.c_size_t, C.c_uint64, C.c_int, C.c_double, C.c_double]
        lib.orc_fill_range.argtypes = [C.c_void_p, C.c_int, C.c_uint64, C.c_size_t, C.c_uint64, C.c_int, C.c_double, C.c_double]
        _port = lib
    return _port


def ref():
    """The compiled reference kernels, or None if oracle/_ref was never built here."""
    global _ref
    if _ref is None and REF_PATH.exists():
        lib = C.CDLL(str(REF_PATH))
        for n in BINARY:
            getattr(lib, f"ref_{n}").argtypes = [_TP, _TP, _TP]
        for n in UNARY:
            getattr(lib, f"ref_{n}").argtypes = [_TP, _TP] + ([C.c_float] if n == "rsqrt" else [])
        lib.ref_scale.argtypes = [_TP, C.POINTER(A.ScalarT), _TP]
        lib.ref_gemm.argtypes = [_TP, _TP, _TP]
        lib.ref_conv2d.argtypes = [_TP, _TP, _TP, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]
        lib.ref_conv2d_bias.argtypes = [_TP, _TP, _TP, _TP, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]
        for n in ("argmax", "argmin", "argsum", "argmean"):
            getattr(lib, f"ref_{n}").argtypes = [_TP, _TP, C.c_uint8]
        lib.ref_cpy.argtypes = [_TP, _TP]
        if hasattr(lib, "ref_conv1d"):
            lib.ref_conv1d.argtypes = [_TP, _TP, _TP, C.c_size_t, C.c_size_t]
            for n in COMPARE:
                getattr(lib, f"ref_{n}").argtypes = [_TP, _TP, _TP]
        lib.ref_allclose.argtypes = [_TP, _TP, C.c_double, C.c_double]
        lib.ref_outer.argtypes = [_TP, _TP, _TP]
        lib.ref_repeat.argtypes = [_TP, _TP, C.c_int, C.c_int]
        lib.ref_concat.argtypes = [_TP, _TP, _TP, C.c_int]
        lib.ref_triu.argtypes = [_TP, _TP, C.c_int]
        lib.ref_tril.argtypes = [_TP, _TP, C.c_int]
        lib.ref_view_as_cartesian.argtypes = [_TP, _TP, _TP]
        lib.ref_view_as_polar.argtypes = [_TP, _TP, _TP]
        _ref = lib
    return _ref


# ---------------------------------------------------------------------------------------
# Convenience layer over CPU torch tensors (torch is used as a typed host buffer only).

from ._records import TN_TO_TORCH, TORCH_TO_TN, broadcast_shape, desc  # noqa: E402
from ._records import matmul_dtype as _matmul_dtype  # noqa: E402


class OracleError(RuntimeError):
    def __init__(self, status):
        super().__init__(A.STATUS_NAMES[status] if 0 <= status < 5 else str(status))
        self.status = status


def _ok(status):
    if status != A.SUCCESS:
        raise OracleError(status)


def fill(shape, dtype: torch.dtype, seed: int, kind: str = "uniform", lo: float = 0.0, hi: float = 1.0,
         first: int = 0, threads: int = 1, pinned: bool = False) -> torch.Tensor:
    """Seeded host tensor: 'uniform' in [lo, hi) (integers: inclusive range), 'normal'(mean=lo, std=hi).
    The generator is counter based (element i depends on (seed, i) only): `first` is the counter of
    the tensor's first element, so a shard of a larger tensor is generated without the rest, and
    `threads` splits the work over host threads without changing a bit of the result."""
    t = torch.empty(tuple(shape), dtype=dtype, pin_memory=pinned)
    n, tn, k = t.numel(), TORCH_TO_TN[dtype], 0 if kind == "uniform" else 1
    es = t.element_size()
    if threads <= 1 or n < (1 << 16):
        _ok(port().orc_fill_range(t.data_ptr(), tn, first, n, seed, k, lo, hi))
        return t
    from concurrent.futures import ThreadPoolExecutor
    bounds = [(n * i) // threads for i in range(threads + 1)]
    lib = port()

    def part(i):
        a, b = bounds[i], bounds[i + 1]
        return lib.orc_fill_range(t.data_ptr() + a * es, tn, first + a, b - a, seed, k, lo, hi)

    with ThreadPoolExecutor(max_workers=threads) as pool:
        for status in pool.map(part, range(threads)):
            _ok(status)
    return t


def _empty(shape, tn):
    return torch.empty(tuple(shape), dtype=TN_TO_TORCH[tn])


def binary(name, a, b, out_dtype=None, impl="port"):
    dt = out_dtype if out_dtype is not None else max(TORCH_TO_TN[a.dtype], TORCH_TO_TN[b.dtype])
    out = _empty(broadcast_shape(a.shape, b.shape), dt)
    da, db, dd = desc(a), desc(b), desc(out)
    if impl == "port":
        _ok(port().orc_binary(BINARY[name], C.byref(da), C.byref(db), C.byref(dd)))
    else:
        _ok(getattr(ref(), f"ref_{name}")(C.byref(da), C.byref(db), C.byref(dd)))
    return out


def unary(name, x, eps=0.0, impl="port"):
    out = _empty(x.shape, TORCH_TO_TN[x.dtype])
    dx, dd = desc(x), desc(out)
    if impl == "port":
        _ok(port().orc_unary(UNARY[name], C.byref(dx), C.byref(dd), eps))
    elif name == "rsqrt":
        _ok(ref().ref_rsqrt(C.byref(dx), C.byref(dd), eps))
    else:
        _ok(getattr(ref(), f"ref_{name}")(C.byref(dx), C.byref(dd)))
    return out


def scale(x, value, impl="port"):
    out = _empty(x.shape, TORCH_TO_TN[x.dtype])
    holder = torch.tensor([value], dtype=x.dtype)
    sc = A.ScalarT(holder.data_ptr(), TORCH_TO_TN[x.dtype])
    dx, dd = desc(x), desc(out)
    fn = port().orc_scale if impl == "port" else ref().ref_scale
    _ok(fn(C.byref(dx), C.byref(sc), C.byref(dd)))
    return out


def matmul(a, b, acc=ACC_WIDE, out_dtype=None, wrap_batch_u8=False, impl="port", out=None):
    batch = broadcast_shape(a.shape[:-2], b.shape[:-2])
    dt = out_dtype if out_dtype is not None else _matmul_dtype(TORCH_TO_TN[a.dtype], TORCH_TO_TN[b.dtype])
    if out is None:
        out = _empty(batch + (a.shape[-2], b.shape[-1]), dt)
    da, db, dd = desc(a), desc(b), desc(out)
    if impl == "port":
        _ok(port().orc_gemm(C.byref(da), C.byref(db), C.byref(dd), acc, int(wrap_batch_u8)))
    else:
        _ok(ref().ref_gemm(C.byref(da), C.byref(db), C.byref(dd)))
    return out


def conv2d(x, w, stride=1, padding=0, bias=None, acc=ACC_WIDE, impl="port"):
    s = (stride, stride) if isinstance(stride, int) else tuple(stride)
    p = (padding, padding) if isinstance(padding, int) else tuple(padding)
    ho = (x.shape[2] + 2 * p[0] - w.shape[2]) // s[0] + 1
    wo = (x.shape[3] + 2 * p[1] - w.shape[3]) // s[1] + 1
    out = _empty((x.shape[0], w.shape[0], ho, wo), TORCH_TO_TN[x.dtype])
    pad, strd = (C.c_size_t * 2)(*p), (C.c_size_t * 2)(*s)
    dx, dw, dd = desc(x), desc(w), desc(out)
    db = desc(bias) if bias is not None else None
    if impl == "port":
        _ok(port().orc_conv2d(C.byref(dx), C.byref(dw), C.byref(db) if db is not None else None, C.byref(dd), pad, strd, acc))
    elif bias is None:
        _ok(ref().ref_conv2d(C.byref(dx), C.byref(dw), C.byref(dd), pad, strd))
    else:
        _ok(ref().ref_conv2d_bias(C.byref(dx), C.byref(dw), C.byref(db), C.byref(dd), pad, strd))
    return out


def conv1d(x, w, stride=1, padding=0, acc=ACC_WIDE, impl="port"):
    """[N, C, L] signal, [Cout, Cin, K] kernel. The restatement is the H = 1 case of conv2d: the
    reference's conv1d loop nest (src/cpu/conv1d.cpp:29-52) visits (ci, kl) in the order conv2d
    visits (ci, kh = 0, kw), so the accumulation order is the same."""
    lo = (x.shape[2] + 2 * padding - w.shape[2]) // stride + 1
    if impl == "port":
        return conv2d(x.unsqueeze(2), w.unsqueeze(2), (1, stride), (0, padding), acc=acc).squeeze(2)
    out = _empty((x.shape[0], w.shape[0], lo), TORCH_TO_TN[x.dtype])
    dx, dw, dd = desc(x), desc(w), desc(out)
    _ok(ref().ref_conv1d(C.byref(dx), C.byref(dw), C.byref(dd), padding, stride))
    return out


def compare(name, a, b, impl="port"):
    """Elementwise comparison -> torch.bool tensor of the broadcast shape (the kernels write it
    bit-packed, element i in bit i % 8 of byte i / 8; `compare_packed` returns those bytes)."""
    packed, shape = compare_packed(name, a, b, impl=impl)
    n = 1
    for s in shape:
        n *= s
    bits = (packed.to(torch.int32).unsqueeze(-1) >> torch.arange(8, dtype=torch.int32)) & 1
    return bits.reshape(-1)[:n].to(torch.bool).reshape(shape)


def compare_packed(name, a, b, impl="port"):
    shape = broadcast_shape(a.shape, b.shape)
    rank = len(shape)
    a = a.reshape((1,) * (rank - a.dim()) + tuple(a.shape))
    b = b.reshape((1,) * (rank - b.dim()) + tuple(b.shape))
    n = 1
    for s in shape:
        n *= s
    packed = torch.full(((n + 7) // 8,), 0xAA, dtype=torch.uint8)  # the kernels must clear what they do not set
    dd = A.TensorT()
    dd.address, dd.rank, dd.dtype, dd.size = packed.data_ptr(), rank, A.BOOLEAN, n
    run = 1
    for i in range(rank - 1, -1, -1):
        dd.shape.sizes[i], dd.strides.sizes[i] = shape[i], run
        run *= shape[i]
    dd.environment.kind, dd.layout = A.HOST, A.CONTIGUOUS
    da, db = desc(a), desc(b)
    if impl == "port":
        _ok(port().orc_compare(COMPARE[name], C.byref(da), C.byref(db), C.byref(dd)))
    else:
        if any(x != y for x, y in zip(a.shape, shape)) or any(x != y for x, y in zip(b.shape, shape)):
            raise ValueError("the reference's comparison kernels take operands of the result's shape")
        _ok(getattr(ref(), f"ref_{name}")(C.byref(da), C.byref(db), C.byref(dd)))
    return packed, shape


def reduce(kind, x, axis=-1, keepdim=False, acc=ACC_WIDE, impl="port"):
    ax = axis + x.dim() if axis < 0 else axis
    shape = list(x.shape)
    if keepdim:
        shape[ax] = 1
    else:
        del shape[ax]
    dt = A.INT64 if kind in ("argmax", "argmin") else TORCH_TO_TN[x.dtype]
    out = _empty(shape, dt)
    dx, dd = desc(x), desc(out)
    if impl == "port":
        _ok(port().orc_reduce(REDUCE[kind], C.byref(dx), C.byref(dd), ax, acc))
    else:
        name = {"sum": "argsum", "mean": "argmean"}.get(kind, kind)
        _ok(getattr(ref(), f"ref_{name}")(C.byref(dx), C.byref(dd), ax))
    return out


# ---- data movement around the path -------------------------------------------------------

def outer(a, b, out_dtype=None, impl="port"):
    """a[i] * b[j]. The restatement is the broadcast multiply of two views, written in the promoted
    dtype; the reference kernel (impl="ref") writes the type of its own table entry, which is wider
    than the promoted one for some pairs, so `out_dtype` must name that type there."""
    if impl == "port":
        return binary("mul", a[:, None], b[None, :], out_dtype=out_dtype)
    dt = out_dtype if out_dtype is not None else max(TORCH_TO_TN[a.dtype], TORCH_TO_TN[b.dtype])
    out = _empty((a.shape[0], b.shape[0]), dt)
    da, db, dd = desc(a), desc(b), desc(out)
    _ok(ref().ref_outer(C.byref(da), C.byref(db), C.byref(dd)))
    return out


def repeat(x, repeats, axis, impl="port"):
    axis = axis % x.dim()
    shape = list(x.shape)
    shape[axis] *= repeats
    out = _empty(shape, TORCH_TO_TN[x.dtype])
    dx, dd = desc(x), desc(out)
    if impl == "port":
        _ok(port().orc_repeat(C.byref(dx), C.byref(dd), axis, repeats))
    else:
        _ok(ref().ref_repeat(C.byref(dx), C.byref(dd), axis, repeats))
    return out


def concat(a, b, axis=0, impl="port"):
    axis = axis % a.dim()
    shape = list(a.shape)
    shape[axis] += b.shape[axis]
    out = _empty(shape, TORCH_TO_TN[a.dtype])
    da, db, dd = desc(a), desc(b), desc(out)
    if impl == "port":
        _ok(port().orc_concat(C.byref(da), C.byref(db), C.byref(dd), axis))
    else:
        _ok(ref().ref_concat(C.byref(da), C.byref(db), C.byref(dd), axis))
    return out


def triangular(x, upper, k=0, impl="port"):
    out = _empty(x.shape, TORCH_TO_TN[x.dtype])
    dx, dd = desc(x), desc(out)
    if impl == "port":
        _ok(port().orc_triangular(C.byref(dx), C.byref(dd), 1 if upper else 0, k))
    else:
        _ok((ref().ref_triu if upper else ref().ref_tril)(C.byref(dx), C.byref(dd), k))
    return out


def complex_pair(a, b, polar, impl="port"):
    wide = torch.float64 in (a.dtype, b.dtype)
    out = _empty(broadcast_shape(a.shape, b.shape), A.COMPLEX128 if wide else A.COMPLEX64)
    rank = out.dim()
    a = a.reshape((1,) * (rank - a.dim()) + tuple(a.shape))
    b = b.reshape((1,) * (rank - b.dim()) + tuple(b.shape))
    da, db, dd = desc(a), desc(b), desc(out)
    if impl == "port":
        _ok(port().orc_complex_pair(C.byref(da), C.byref(db), C.byref(dd), 1 if polar else 0))
    else:
        _ok((ref().ref_view_as_polar if polar else ref().ref_view_as_cartesian)(C.byref(da), C.byref(db), C.byref(dd)))
    return out
