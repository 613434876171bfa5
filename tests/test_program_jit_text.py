"""The device headers that the library hands to the run-time compiler must compile under NVRTC for
sm_100a without a GPU: this is the same translation unit eltwise_jit.cu builds for a caller's node list,
compiled here with the NVRTC of the CUDA toolkit. Skipped where no libnvrtc can be loaded."""
import ctypes as C
import re
from pathlib import Path

import pytest

from tannic_b200 import _abi as A

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "tannic_b200" / "csrc"
CUDA_INCLUDE = Path("/usr/local/cuda/include")


def load_nvrtc():
    for name in ("libnvrtc.so.12", "libnvrtc.so", "/usr/local/cuda/lib64/libnvrtc.so.12", "/usr/local/cuda/lib64/libnvrtc.so"):
        try:
            return C.CDLL(name)
        except OSError:
            continue
    return None


def opcode_defines():
    header = (ROOT / "include" / "tannic_b200.h").read_text()
    body = re.search(r"typedef enum tn_eltwise_opcode \{([^}]*)\} tn_eltwise_opcode;", header).group(1)
    names = [t.split("=")[0].strip() for t in body.replace("\n", " ").split(",") if t.strip()]
    names = [n for n in names if n != "TN_OP_COUNT"]
    assert names[0] == "TN_OP_ADD" and names.index("TN_OP_SCALE") == A.OP_SCALE and names.index("TN_OP_TANH") == A.OP_TANH
    return [f"-D{n}={i}" for i, n in enumerate(names)] + ["-DTN_PROGRAM_MAX_INPUTS=4", "-DTN_PROGRAM_MAX_NODES=16"]


@pytest.mark.parametrize("ctype", ["__half", "__nv_bfloat16", "float", "double"])
@pytest.mark.parametrize("scalar", ["false", "true"])
def test_program_template_compiles_under_nvrtc(ctype, scalar):
    rtc = load_nvrtc()
    if rtc is None or not (CUDA_INCLUDE / "cuda_fp16.h").exists():
        pytest.skip("no NVRTC or CUDA headers on this machine")
    nodes = [(A.OP_MUL, 0, 1), (A.OP_ADD, 4, 0), (A.OP_TANH, 5, 5), (A.OP_SCALE, 6, 6), (A.OP_RSQRT, 0, 0), (A.OP_SUB, 7, 8),
             (A.OP_POW, 9, 1), (A.OP_LOG, 10, 10), (A.OP_SIN, 11, 11), (A.OP_ABS, 12, 12)]
    text = ", ".join("{%d, %d, %d}" % n for n in nodes)
    source = ('#include "eltwise_program.cuh"\nnamespace tnb { namespace prog {\nstruct ProgJit {\n'
              f"    static constexpr int N = {len(nodes)};\n    static constexpr int NIN = 2;\n"
              f"    static constexpr NodeSpec nodes[N] = {{{text}}};\n}};\n}} }}\n").encode()
    headers = [(CSRC / "numeric.cuh").read_bytes(), (CSRC / "eltwise_program.cuh").read_bytes()]
    names = [b"numeric.cuh", b"eltwise_program.cuh"]
    prog = C.c_void_p()
    assert rtc.nvrtcCreateProgram(C.byref(prog), source, b"tn_program.cu", 2, (C.c_char_p * 2)(*headers), (C.c_char_p * 2)(*names)) == 0
    unroll = "1" if scalar == "true" else "2"
    expr = f"tnb::prog::ew_program_rows<{ctype}, tnb::prog::ProgJit, {unroll}, {scalar}>".encode()
    assert rtc.nvrtcAddNameExpression(prog, expr) == 0
    options = [b"--gpu-architecture=sm_100a", b"-std=c++17", b"-I" + str(CUDA_INCLUDE).encode()] + [d.encode() for d in opcode_defines()]
    rc = rtc.nvrtcCompileProgram(prog, len(options), (C.c_char_p * len(options))(*options))
    size = C.c_size_t()
    rtc.nvrtcGetProgramLogSize(prog, C.byref(size))
    log = C.create_string_buffer(size.value or 1)
    rtc.nvrtcGetProgramLog(prog, log)
    assert rc == 0, log.value.decode(errors="replace")[:4000]
    lowered = C.c_char_p()
    assert rtc.nvrtcGetLoweredName(prog, expr, C.byref(lowered)) == 0 and lowered.value.startswith(b"_ZN3tnb4prog15ew_program_rows")
    cubin = C.c_size_t()
    assert rtc.nvrtcGetCUBINSize(prog, C.byref(cubin)) == 0 and cubin.value > 1000
    rtc.nvrtcDestroyProgram(C.byref(prog))
