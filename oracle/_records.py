"""TEST INFRASTRUCTURE — the oracle's own view of the reference's argument records and front-end rules.

Kept separate from the product package on purpose: the checker must not share the dtype-promotion,
broadcast or record-layout code with the thing it checks. The records follow the reference's
include/tannic/runtime/tensor.h:37-73, types.h:29-44, status.h:26-32 and resources.h:35-59; the
rules follow include/tannic/operations.hpp:133-152 (result dtype = larger enum value, NumPy
broadcast) and include/tannic/transformations.hpp:87-152 (matmul result dtype).
"""
from __future__ import annotations

import ctypes as C

import torch

MAX_RANK = 8
ANY, BOOLEAN, INT8, INT16, INT32, INT64, FLOAT16, BFLOAT16, FLOAT32, FLOAT64, COMPLEX64, COMPLEX128, UNKNOWN, TYPES = range(14)
SUCCESS, ERROR, UNSUPPORTED_DTYPE, NULL_ALLOCATOR, INCOMPATIBLE_DEVICES = range(5)
STATUS_NAMES = ["SUCCESS", "ERROR", "UNSUPPORTED_DTYPE", "NULL_ALLOCATOR", "INCOMPATIBLE_DEVICES"]
SINGLETON, CONTIGUOUS, STRIDED = range(3)
HOST, DEVICE = 0, 1
PAGEABLE, PINNED = 1, 2


class _Resource(C.Union):
    _fields_ = [("host_traits", C.c_int), ("device_id", C.c_int)]


class Environment(C.Structure):
    _fields_ = [("kind", C.c_int), ("resource", _Resource)]


class Shape(C.Union):
    _fields_ = [("address", C.c_void_p), ("sizes", C.c_size_t * MAX_RANK)]


class Strides(C.Union):
    _fields_ = [("address", C.c_void_p), ("sizes", C.c_int64 * MAX_RANK)]


class TensorT(C.Structure):
    _fields_ = [("address", C.c_void_p), ("rank", C.c_uint8), ("shape", Shape), ("strides", Strides), ("dtype", C.c_int),
                ("environment", Environment), ("size", C.c_size_t), ("layout", C.c_int)]


class ScalarT(C.Structure):
    _fields_ = [("address", C.c_void_p), ("dtype", C.c_int)]


TORCH_TO_TN = {
    torch.int8: INT8, torch.int16: INT16, torch.int32: INT32, torch.int64: INT64,
    torch.float16: FLOAT16, torch.bfloat16: BFLOAT16, torch.float32: FLOAT32, torch.float64: FLOAT64,
    torch.complex64: COMPLEX64, torch.complex128: COMPLEX128,
}
TN_TO_TORCH = {v: k for k, v in TORCH_TO_TN.items()}


def desc(t: torch.Tensor) -> TensorT:
    """Host tensor record over a CPU torch tensor (torch is a typed host buffer here)."""
    if t.is_cuda:
        raise ValueError("the oracle runs on host tensors")
    r = TensorT()
    r.address = t.data_ptr()
    r.rank = t.dim()
    size = 1
    for i, (n, s) in enumerate(zip(t.shape, t.stride())):
        r.shape.sizes[i] = n
        r.strides.sizes[i] = s
        size *= n
    r.dtype = TORCH_TO_TN[t.dtype]
    r.environment.kind = HOST
    r.environment.resource.host_traits = PINNED if t.is_pinned() else PAGEABLE
    r.size = size
    expect, dense = 1, True
    for n, s in zip(reversed(t.shape), reversed(t.stride())):
        dense = dense and s == expect
        expect *= n
    r.layout = SINGLETON if size == 1 else (CONTIGUOUS if dense else STRIDED)
    return r


def broadcast_shape(a, b) -> tuple:
    """include/tannic/operations.hpp:137-152: trailing-aligned, extent 1 stretches."""
    a, b = tuple(a), tuple(b)
    n = max(len(a), len(b))
    a, b = (1,) * (n - len(a)) + a, (1,) * (n - len(b)) + b
    out = []
    for x, y in zip(a, b):
        if x != y and 1 not in (x, y):
            raise ValueError("Shapes are not broadcast-compatible.")
        out.append(x if y == 1 else y)
    return tuple(out)


_INTS = (INT8, INT16, INT32, INT64)
_HALVES = (FLOAT16, BFLOAT16)


def matmul_dtype(a: int, b: int) -> int:
    """include/tannic/transformations.hpp:87-152, written as the table's rows."""
    if a in _INTS and b in _INTS:
        return INT64 if (INT64 in (a, b) or a == b == INT32) else INT32
    if a in _HALVES or b in _HALVES:
        h, o = (a, b) if a in _HALVES else (b, a)
        if o == h:
            return h
        if o in _HALVES:
            return FLOAT16
        if o in (INT8, INT16):
            return h
        if o in (INT32, FLOAT32):
            return FLOAT32
        if o in (INT64, FLOAT64):
            return FLOAT64
    if FLOAT64 in (a, b):
        return FLOAT64
    if FLOAT32 in (a, b) and a in (FLOAT32, INT32) and b in (FLOAT32, INT32):
        return FLOAT32
    raise ValueError("Unsuported dtypes")
