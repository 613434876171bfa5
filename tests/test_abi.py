"""CPU-side checks of the drop-in boundary: the header compiles as C and C++, the library exports
every symbol the header declares, the ctypes records match the C layout, and the entry points
refuse host tensors (no CPU fallback) — all without a GPU and without any compute call."""
import ctypes as C
import re
import subprocess
from pathlib import Path

import pytest
import torch

from tannic_b200 import _abi as A
from tannic_b200 import ops as tb

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "tannic_b200.h"


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(tn_[a-z0-9_]+)\s*\(", text)))


def test_header_compiles_as_c_and_cxx(tmp_path):
    c = tmp_path / "t.c"
    c.write_text('#include "tannic_b200.h"\nint main(void) { tn_tensor_t t; (void)t; return (int)sizeof(tn_tensor_t) == 0; }\n')
    subprocess.run(["gcc", "-std=c11", "-Wall", "-Werror", "-fsyntax-only", f"-I{HEADER.parent}", str(c)], check=True)
    cxx = tmp_path / "t.cpp"
    cxx.write_text('#include "tannic_b200.h"\nstatic_assert(sizeof(tn_tensor_t) == 176, "layout");\nint main() { return 0; }\n')
    subprocess.run(["g++", "-std=c++17", "-Wall", "-Werror", "-fsyntax-only", f"-I{HEADER.parent}", str(cxx)], check=True)


def test_library_exports_every_declared_symbol():
    lib = A.lib()
    names = declared_functions()
    assert len(names) >= 45
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    # and the ctypes prototypes cover the header
    assert set(names) == set(A.PROTOTYPES), set(names) ^ set(A.PROTOTYPES)


def test_ctypes_records_match_the_c_layout(tmp_path):
    src = tmp_path / "layout.c"
    src.write_text(r'''
#include <stdio.h>
#include <stddef.h>
#include "tannic_b200.h"
int main(void) {
    printf("%zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu\n", sizeof(tn_tensor_t), offsetof(tn_tensor_t, rank),
           offsetof(tn_tensor_t, shape), offsetof(tn_tensor_t, strides), offsetof(tn_tensor_t, dtype),
           offsetof(tn_tensor_t, environment), offsetof(tn_tensor_t, size), offsetof(tn_tensor_t, layout),
           sizeof(tn_scalar_t), sizeof(tn_stream_t), sizeof(tn_eltwise_node_t), offsetof(tn_eltwise_node_t, imm));
    return 0;
}''')
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-std=c11", f"-I{HEADER.parent}", str(src), "-o", str(exe)], check=True)
    got = [int(x) for x in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()]
    T = A.TensorT
    want = [C.sizeof(T), T.rank.offset, T.shape.offset, T.strides.offset, T.dtype.offset, T.environment.offset, T.size.offset,
            T.layout.offset, C.sizeof(A.ScalarT), C.sizeof(A.StreamT), C.sizeof(A.EltwiseNode), A.EltwiseNode.imm.offset]
    assert got == want


def test_dtype_sizes_and_error_text():
    lib = A.lib()
    for dt, size in A.DTYPE_SIZE.items():
        assert lib.tn_dtype_size(dt) == size
    assert lib.tn_dtype_size(A.ANY) == 0 and lib.tn_dtype_size(A.UNKNOWN) == 0
    assert isinstance(lib.tn_last_error(), bytes)


def test_host_tensors_are_refused_not_computed():
    a = torch.ones(4)
    out = torch.zeros(4)
    da, dd = tb.desc(a), tb.desc(out)
    lib = A.lib()
    assert lib.tn_add(C.byref(da), C.byref(da), C.byref(dd), A.StreamT(0)) == A.INCOMPATIBLE_DEVICES
    assert b"host" in lib.tn_last_error() or b"device" in lib.tn_last_error()
    assert lib.tn_log(C.byref(da), C.byref(dd), A.StreamT(0)) == A.INCOMPATIBLE_DEVICES
    assert lib.tn_gemm(C.byref(tb.desc(torch.ones(2, 2))), C.byref(tb.desc(torch.ones(2, 2))), C.byref(tb.desc(torch.ones(2, 2))), A.StreamT(0)) == A.INCOMPATIBLE_DEVICES
    assert torch.equal(out, torch.zeros(4))  # nothing was computed on the host
    # dtype errors are reported before anything else
    h, b = tb.desc(torch.ones(4, dtype=torch.float16)), tb.desc(torch.ones(4, dtype=torch.bfloat16))
    assert lib.tn_add(C.byref(h), C.byref(b), C.byref(dd), A.StreamT(0)) == A.UNSUPPORTED_DTYPE
    assert lib.tn_argmean(C.byref(tb.desc(torch.ones(4, dtype=torch.int32))), C.byref(dd), A.StreamT(0), 0) == A.UNSUPPORTED_DTYPE


def test_process_wide_switches_validate_their_arguments():
    """Settings and counters that need no device: the SM margin, the run-time compiler's mode, the path counters."""
    lib = A.lib()
    assert lib.tn_set_sm_margin(65) == A.ERROR and b"0..64" in lib.tn_last_error()
    assert lib.tn_set_sm_margin(-1) == A.ERROR
    assert lib.tn_set_sm_margin(0) == A.SUCCESS
    assert lib.tn_program_jit_enable(3) == A.ERROR
    assert lib.tn_program_jit_enable(1) == A.SUCCESS
    sentinel = 2 ** 63
    counts = (C.c_uint64 * 4)(sentinel, sentinel, sentinel, sentinel)
    assert lib.tn_gemm_path_launches(counts) == A.SUCCESS and all(c < sentinel for c in counts)  # all four were written
    stats = tb.program_jit_stats()
    assert set(stats) == {"compiled", "failed", "available", "from_disk", "log"}
    # mirrors and packed weights are checked before any device work
    t = tb.desc(torch.ones(2, 2, dtype=torch.bfloat16))
    assert lib.tn_gemm_mirrored(C.byref(t), C.byref(t), C.byref(t), None, 8, A.StreamT(0)) == A.ERROR
    n = C.c_size_t(7)
    w = tb.desc(torch.ones(4, 3, 3, 3, dtype=torch.float16))
    assert lib.tn_conv2d_packed_weights_size(C.byref(w), C.byref(n)) == A.SUCCESS and n.value == 3 * 3 * 4 * 8 * 2
    w32 = tb.desc(torch.ones(4, 3, 3, 3, dtype=torch.float32))
    assert lib.tn_conv2d_packed_weights_size(C.byref(w32), C.byref(n)) == A.SUCCESS and n.value == 0


def test_front_end_rules_mirror_the_reference():
    # NumPy broadcast, include/tannic/operations.hpp:137-152
    assert tb.broadcast_shape((2, 1, 3), (1, 4, 3)) == (2, 4, 3)
    assert tb.broadcast_shape((5, 7), (7,)) == (5, 7)
    assert tb.broadcast_shape((), (3,)) == (3,)
    with pytest.raises(ValueError):
        tb.broadcast_shape((2, 3), (4, 3))
    # matmul promotion table, include/tannic/transformations.hpp:87-152
    m = tb._matmul_dtype
    assert m(A.INT8, A.INT8) == A.INT32 and m(A.INT32, A.INT32) == A.INT64 and m(A.INT16, A.INT64) == A.INT64
    assert m(A.FLOAT16, A.FLOAT16) == A.FLOAT16 and m(A.BFLOAT16, A.BFLOAT16) == A.BFLOAT16
    assert m(A.BFLOAT16, A.FLOAT16) == A.FLOAT16 and m(A.FLOAT16, A.INT8) == A.FLOAT16
    assert m(A.INT32, A.BFLOAT16) == A.FLOAT32 and m(A.FLOAT16, A.INT64) == A.FLOAT64
    assert m(A.FLOAT32, A.FLOAT32) == A.FLOAT32 and m(A.FLOAT32, A.FLOAT64) == A.FLOAT64 and m(A.INT32, A.FLOAT32) == A.FLOAT32
    # layout hint, include/tannic/tensor.hpp:61-69,118-124
    t = torch.zeros(3, 4)
    assert tb.desc(t).layout == A.CONTIGUOUS and tb.desc(t.t()).layout == A.STRIDED and tb.desc(torch.zeros(1, 1)).layout == A.SINGLETON
    d = tb.desc(t.t())
    assert (d.rank, d.size, list(d.shape.sizes[:2]), list(d.strides.sizes[:2])) == (2, 12, [4, 3], [1, 4])
    assert d.environment.kind == A.HOST


def test_header_is_plain_c(tmp_path):
    """include/tannic_b200.h compiles as C11 on its own (no C++ or CUDA types leak into the ABI), and a C
    translation unit that takes the address of every declared entry point links against the library."""
    import re
    import shutil
    import subprocess
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    gcc = shutil.which("gcc")
    lib = root / "tannic_b200" / "libtannic_b200.so"
    if gcc is None or not lib.exists():
        pytest.skip("needs gcc and the built library")
    header = (root / "include" / "tannic_b200.h").read_text()
    names = sorted(set(re.findall(r"\b(tn_[a-z0-9_]+)\s*\(", header)))
    assert len(names) > 50
    src = tmp_path / "abi.c"
    src.write_text('#include "tannic_b200.h"\n#include <stdio.h>\ntypedef void (*any_fn)(void);\nint main(void) {\n  any_fn table[] = {\n'
                   + "".join(f"    (any_fn){n},\n" for n in names)
                   + '  };\n  printf("%zu\\n", sizeof table / sizeof table[0]);\n  return sizeof(tn_tensor_t) == 176 ? 0 : 1;\n}\n')
    exe = tmp_path / "abi"
    subprocess.run([gcc, "-std=c11", "-Wall", "-Werror", "-pedantic", f"-I{root / 'include'}", str(src), "-o", str(exe),
                    f"-L{lib.parent}", "-ltannic_b200", f"-Wl,-rpath,{lib.parent}"], check=True, capture_output=True, text=True)
