"""ctypes view of include/tannic_b200.h: the records, the enums and the loaded library.

The product path has no fallback: if libtannic_b200.so is missing, `lib()` raises.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libtannic_b200.so"

MAX_RANK = 8

# tn_dtype (same values as the reference's `enum type`, include/tannic/runtime/types.h:29-44)
ANY, BOOLEAN, INT8, INT16, INT32, INT64, FLOAT16, BFLOAT16, FLOAT32, FLOAT64, COMPLEX64, COMPLEX128, UNKNOWN, TYPES = range(14)
DTYPE_NAMES = ["any", "boolean", "int8", "int16", "int32", "int64", "float16", "bfloat16", "float32", "float64",
               "complex64", "complex128", "unknown"]
DTYPE_SIZE = {BOOLEAN: 1, INT8: 1, INT16: 2, INT32: 4, INT64: 8, FLOAT16: 2, BFLOAT16: 2, FLOAT32: 4, FLOAT64: 8,
              COMPLEX64: 8, COMPLEX128: 16}

# tn_status
SUCCESS, ERROR, UNSUPPORTED_DTYPE, NULL_ALLOCATOR, INCOMPATIBLE_DEVICES = range(5)
STATUS_NAMES = ["SUCCESS", "ERROR", "UNSUPPORTED_DTYPE", "NULL_ALLOCATOR", "INCOMPATIBLE_DEVICES"]

SINGLETON, CONTIGUOUS, STRIDED = range(3)
HOST, DEVICE = 0, 1
PAGEABLE, PINNED = 1, 2

# tn_eltwise_opcode
(OP_ADD, OP_SUB, OP_MUL, OP_POW, OP_NEG, OP_LOG, OP_EXP, OP_SQRT, OP_RSQRT, OP_ABS, OP_SIN, OP_COS, OP_TAN,
 OP_SINH, OP_COSH, OP_TANH, OP_SCALE) = range(17)


class _Resource(C.Union):
    _fields_ = [("host_traits", C.c_int), ("device_id", C.c_int)]


class Environment(C.Structure):
    _fields_ = [("kind", C.c_int), ("resource", _Resource)]


class Shape(C.Union):
    _fields_ = [("address", C.c_void_p), ("sizes", C.c_size_t * MAX_RANK)]


class Strides(C.Union):
    _fields_ = [("address", C.c_void_p), ("sizes", C.c_int64 * MAX_RANK)]


class TensorT(C.Structure):
    _fields_ = [
        ("address", C.c_void_p),
        ("rank", C.c_uint8),
        ("shape", Shape),
        ("strides", Strides),
        ("dtype", C.c_int),
        ("environment", Environment),
        ("size", C.c_size_t),
        ("layout", C.c_int),
    ]


class ScalarT(C.Structure):
    _fields_ = [("address", C.c_void_p), ("dtype", C.c_int)]


class StreamT(C.Structure):
    _fields_ = [("address", C.c_size_t)]


class DeviceT(C.Structure):
    _fields_ = [("id", C.c_int)]


class EltwiseNode(C.Structure):
    _fields_ = [("opcode", C.c_uint8), ("lhs", C.c_uint8), ("rhs", C.c_uint8), ("imm", C.c_float)]


class TannicError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"{STATUS_NAMES[status] if 0 <= status < 5 else status}: {message}")
        self.status = status


_TP = C.POINTER(TensorT)
_UNARY = ["neg", "repack", "log", "exp", "sqrt", "abs", "sin", "cos", "tan", "sinh", "cosh", "tanh"]
_BINARY = ["add", "sub", "mul", "pow", "eq", "ne", "gt", "ge", "lt", "le"]
_REDUCE = ["argmax", "argmin", "argsum", "argmean", "max"]

# name -> argtypes (restype is tn_status unless listed in _RESTYPES)
PROTOTYPES = {
    "tn_dtype_size": [C.c_int],
    "tn_last_error": [],
    "tn_device_count": [C.POINTER(C.c_int)],
    "tn_set_device": [C.c_int],
    "tn_stream_pop": [C.POINTER(DeviceT), C.POINTER(StreamT)],
    "tn_stream_put": [C.POINTER(DeviceT), StreamT],
    "tn_stream_synchronize": [StreamT],
    "tn_allocate": [C.POINTER(DeviceT), C.c_size_t, C.POINTER(C.c_void_p)],
    "tn_deallocate": [C.POINTER(DeviceT), C.c_void_p],
    "tn_copy_from_host": [C.POINTER(DeviceT), C.c_void_p, C.c_void_p, C.c_size_t],
    "tn_copy_to_host": [C.POINTER(DeviceT), C.c_void_p, C.c_void_p, C.c_size_t],
    "tn_assign_from_host": [C.POINTER(DeviceT), C.c_void_p, C.c_void_p, C.c_size_t],
    "tn_flush_assignments": [],
    "tn_h2d_copy_count": [],
    "tn_copy_from_host_async": [C.POINTER(DeviceT), C.c_void_p, C.c_void_p, C.c_size_t, StreamT],
    "tn_copy_to_host_async": [C.POINTER(DeviceT), C.c_void_p, C.c_void_p, C.c_size_t, StreamT],
    "tn_compare_from_host": [C.POINTER(DeviceT), C.c_void_p, C.c_void_p, C.c_size_t, C.POINTER(C.c_int)],
    "tn_copy": [_TP, _TP, C.c_size_t, StreamT],
    "tn_host_allocate_pinned": [C.c_size_t, C.POINTER(C.c_void_p)],
    "tn_host_free_pinned": [C.c_void_p],
    "tn_host_memory_nodes": [],
    "tn_device_numa_node": [C.POINTER(DeviceT), C.POINTER(C.c_int)],
    "tn_host_allocate_pinned_near": [C.POINTER(DeviceT), C.c_size_t, C.POINTER(C.c_void_p)],
    "tn_bind_thread_near": [C.POINTER(DeviceT), C.POINTER(C.c_int)],
    "tn_program_jit_enable": [C.c_int],
    "tn_program_jit_stats": [C.POINTER(C.c_uint), C.POINTER(C.c_uint), C.POINTER(C.c_uint), C.POINTER(C.c_uint)],
    "tn_eltwise_program_host": [C.POINTER(DeviceT), C.POINTER(_TP), C.c_int, C.POINTER(EltwiseNode), C.c_int, _TP, C.c_int],
    "tn_gemm_scaled_stats": [_TP, _TP, C.POINTER(ScalarT), _TP, _TP, _TP, _TP, StreamT],
    "tn_rsqrt": [_TP, _TP, StreamT, C.c_float],
    "tn_scale": [_TP, C.POINTER(ScalarT), _TP, StreamT],
    "tn_eltwise_program": [C.POINTER(_TP), C.c_int, C.POINTER(EltwiseNode), C.c_int, _TP, StreamT],
    "tn_gemm": [_TP, _TP, _TP, StreamT],
    "tn_gemm_scaled": [_TP, _TP, C.POINTER(ScalarT), _TP, StreamT],
    "tn_conv2d": [_TP, _TP, _TP, StreamT, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)],
    "tn_conv2d_bias": [_TP, _TP, _TP, _TP, StreamT, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)],
    "tn_conv2d_packed_weights_size": [_TP, C.POINTER(C.c_size_t)],
    "tn_conv2d_pack_weights": [_TP, C.c_void_p, StreamT],
    "tn_conv2d_prepacked": [_TP, _TP, C.c_void_p, _TP, _TP, StreamT, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)],
    "tn_conv1d": [_TP, _TP, _TP, StreamT, C.c_size_t, C.c_size_t],
    "tn_outer": [_TP, _TP, _TP, StreamT],
    "tn_repeat": [_TP, _TP, C.c_int, C.c_int, StreamT],
    "tn_concat": [_TP, _TP, _TP, StreamT, C.c_int],
    "tn_triu": [_TP, _TP, StreamT, C.c_int],
    "tn_tril": [_TP, _TP, StreamT, C.c_int],
    "tn_view_as_cartesian": [_TP, _TP, _TP, StreamT],
    "tn_view_as_polar": [_TP, _TP, _TP, StreamT],
    "tn_reduce_stats": [_TP, _TP, _TP, _TP, StreamT, C.c_uint8],
    "tn_argsum_fixed_scratch": [_TP, _TP, StreamT, C.c_uint8],
    "tn_cpy": [_TP, _TP, StreamT],
    "tn_allclose": [_TP, _TP, StreamT, C.c_double, C.c_double, C.POINTER(C.c_int)],
    "tn_device_errors": [C.POINTER(C.c_uint)],
    "tn_selftest_bounded_wait": [C.POINTER(DeviceT), StreamT, C.c_uint],
    "tn_launch_count": [],
    "tn_gemm_mirrored": [_TP, _TP, _TP, C.POINTER(_TP), C.c_int, StreamT],
    "tn_set_sm_margin": [C.c_int],
    "tn_gemm_path_launches": [C.POINTER(C.c_uint64)],
    "tn_program_jit_log": [],
}
for _n in _UNARY:
    PROTOTYPES[f"tn_{_n}"] = [_TP, _TP, StreamT]
for _n in _BINARY:
    PROTOTYPES[f"tn_{_n}"] = [_TP, _TP, _TP, StreamT]
for _n in _REDUCE:
    PROTOTYPES[f"tn_{_n}"] = [_TP, _TP, StreamT, C.c_uint8]

_RESTYPES = {"tn_dtype_size": C.c_size_t, "tn_last_error": C.c_char_p, "tn_program_jit_log": C.c_char_p, "tn_launch_count": C.c_uint64, "tn_h2d_copy_count": C.c_uint64}


def bind(cdll: C.CDLL, names=None) -> C.CDLL:
    """Attach argtypes / restype of every declared entry point; raises if a symbol is missing."""
    for name, argtypes in PROTOTYPES.items():
        if names is not None and name not in names:
            continue
        fn = getattr(cdll, name)  # AttributeError if the library does not export it
        fn.argtypes = argtypes
        fn.restype = _RESTYPES.get(name, C.c_int)
    return cdll


_lib = None


def lib() -> C.CDLL:
    """The CUDA backend. There is no CPU fallback: a missing library is an error."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m tannic_b200.build` "
                "(the device path has no CPU fallback)")
        _lib = bind(C.CDLL(str(LIB_PATH), mode=os.RTLD_GLOBAL if hasattr(os, "RTLD_GLOBAL") else 0))
    return _lib


def check(status: int) -> None:
    if status != SUCCESS:
        raise TannicError(status, lib().tn_last_error().decode(errors="replace"))


def make_tensor(address: int, shape, strides, dtype: int, device: int | None, pinned: bool = False) -> TensorT:
    """Fill a tn_tensor_t the way the reference's Node does (src/graph.cpp:9-64)."""
    t = TensorT()
    t.address = address
    t.rank = len(shape)
    size = 1
    for i, (n, s) in enumerate(zip(shape, strides)):
        t.shape.sizes[i] = n
        t.strides.sizes[i] = s
        size *= n
    t.dtype = dtype
    if device is None:
        t.environment.kind = HOST
        t.environment.resource.host_traits = PINNED if pinned else PAGEABLE
    else:
        t.environment.kind = DEVICE
        t.environment.resource.device_id = device
    t.size = size
    # layout hint as the reference computes it (include/tannic/tensor.hpp:61-69,118-124,
    # src/bindings.cpp:96): one element -> SINGLETON; exact row-major strides -> CONTIGUOUS
    expect, contiguous = 1, True
    for n, s in zip(reversed(shape), reversed(strides)):
        if s != expect:
            contiguous = False
        expect *= n
    t.layout = SINGLETON if size == 1 else (CONTIGUOUS if contiguous else STRIDED)
    return t
