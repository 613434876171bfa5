"""The literal tensors of the reference's own tests (tests/golden/reference_vectors.json, extracted
from tests/cpu/*.cpp of the reference by tests/golden/extract_reference_vectors.py) replayed on

  * the C restatement (oracle/tannic_oracle.c)            — CPU, pins the oracle;
  * the CUDA path through the C ABI                        — marked gpu, like tests/cuda/*.cpp of the
                                                             reference, which repeat the CPU cases on Device().

What each test does with its tensors is written here by hand, with the reference line it mirrors.
Comparison is the reference's own `allclose` rule, |a-b| <= atol + rtol*|b| with its defaults
rtol 1e-5 / atol 1e-8 (include/tannic/comparisons.hpp:128) unless the test passes its own.
"""
import json
import math
from pathlib import Path

import pytest
import torch

import oracle

VECTORS = json.loads((Path(__file__).parent / "golden" / "reference_vectors.json").read_text())
DT = {"float32": torch.float32, "int32": torch.int32, "float64": torch.float64}


def tensors(name):
    entry = VECTORS[name]
    return {k: torch.tensor(v["values"], dtype=DT[v["dtype"]]).reshape(v["shape"]) for k, v in entry["tensors"].items()}, entry.get("asserts", [])


class CpuBackend:
    """The C restatement, storage-type accumulation (= the literal reference CPU behaviour)."""
    name = "port"

    def up(self, t): return t
    def down(self, t): return t
    def matmul(self, a, b): return oracle.matmul(a, b, acc=oracle.ACC_STORAGE)
    def binary(self, op, a, b): return oracle.binary(op, a, b)
    def unary(self, op, x, eps=0.0): return oracle.unary(op, x, eps=eps)
    def conv(self, x, w, stride, pad, bias=None): return oracle.conv2d(x, w, stride, pad, bias=bias, acc=oracle.ACC_STORAGE)
    def conv1d(self, x, w, stride, pad): return oracle.conv1d(x, w, stride, pad, acc=oracle.ACC_STORAGE)
    def reduce(self, kind, x, axis, keepdim=False): return oracle.reduce(kind, x, axis, keepdim, acc=oracle.ACC_STORAGE)


class GpuBackend:
    name = "cuda"

    def __init__(self):
        from tannic_b200 import ops
        self.tb = ops

    def up(self, t): return t.cuda()
    def down(self, t): return t.cpu()
    def matmul(self, a, b): return self.tb.matmul(a, b)
    def binary(self, op, a, b): return getattr(self.tb, op)(a, b)
    def unary(self, op, x, eps=0.0): return self.tb.rsqrt(x, eps) if op == "rsqrt" else getattr(self.tb, op)(x)
    def conv(self, x, w, stride, pad, bias=None): return self.tb.convolve2D(x, w, stride, pad, bias=bias)
    def conv1d(self, x, w, stride, pad): return self.tb.convolve1D(x, w, stride, pad)
    def reduce(self, kind, x, axis, keepdim=False): return getattr(self.tb, kind)(x, axis, keepdim)


def allclose(got, want, rtol=1e-5, atol=1e-8):
    g, w = got.double(), want.double()
    # the reference flags an element only when `fabs(a - b) > atol + rtol * fabs(b)` is true
    # (src/cpu/val.cpp:33), so inf vs inf (difference NaN) passes
    return got.shape == want.shape and not bool(((g - w).abs() > atol + rtol * w.abs()).any())


def check_asserts(asserts, named):
    for name, index, value in asserts:
        if name not in named:
            continue
        t = named[name]
        for i in index:
            t = t[i]
        assert float(t) == pytest.approx(value, rel=1e-6, abs=1e-3 if name == "data" else 0.0), (name, index, float(t), value)


def run_case(case, be):
    t, asserts = tensors(case)
    up, down = be.up, be.down
    suite, name = case.split(".")
    if suite == "MatmulTests":
        # tests/cpu/test-matmul.cpp:12-238
        a = up(t["A"] if "A" in t else t["X"])
        b = up(t["B"] if "B" in t else t["Y"])
        if name in ("SecondTransposed", "Rank4_SecondTransposed", "Rank4Rank2StridedTransposed"):
            b = b.transpose(-1, -2)
        if name == "BothTransposed":
            a, b = a.transpose(-1, -2), b.transpose(-1, -2)
        assert allclose(down(be.matmul(a, b)), t["Z_expected"])
    elif suite == "TestUnaryOp":
        assert allclose(down(be.unary("neg", up(t["A"]))), t["expected"])  # test-operations.cpp:11-28
    elif suite == "TestBinaryOps":
        if name in ("Addition", "Multiplication", "Subtraction"):  # test-operations.cpp:30-109, [2,1,3] (+) [1,4,3]
            op = {"Addition": "add", "Multiplication": "mul", "Subtraction": "sub"}[name]
            assert allclose(down(be.binary(op, up(t["A"]), up(t["B"]))), t["expected"])
        elif name == "Power":  # test-operations.cpp:131-158: expectation is std::pow of the same operands
            got = down(be.binary("pow", up(t["A"]), up(t["B"])))
            want = torch.pow(t["A"].double().expand(2, 4, 3), t["B"].double().expand(2, 4, 3)).float()
            assert allclose(got, want)
        elif name == "BroadcastMultiplyAdd":  # test-operations.cpp:160-181, X * W + b with rtol 1e-5
            got = be.binary("add", be.binary("mul", up(t["X"]), up(t["W"])), up(t["b"]))
            assert allclose(down(got), t["expected"], rtol=1e-5, atol=1e-5)
        else:
            pytest.skip("complex dtypes are outside the path")
    elif suite in ("TestConvolution", "BiasedConvolution"):
        # tests/cpu/test-convolutions.cpp:130-491
        x = up(t["input"] if "input" in t else t["X"])
        w = up(t["kernel"] if "kernel" in t else t["K"])
        stride, pad = {"Simple2D": (1, 0), "Stride2": (2, 0), "Padding1": (1, 1), "MultiChannelInput": (1, 0), "Kernel1x1": (1, 0)}.get(name, (1, 1))
        bias = None
        if name == "BigBiasedCong":
            bias = up(torch.tensor([10.0]))
        if name == "BigBiasedConv2OutChannels":
            bias = up(torch.tensor([10.0, -5.0]))
        got = down(be.conv(x, w, stride, pad, bias=bias))
        want = t.get("expected", t.get("Y_expected"))
        if want is not None:
            assert allclose(got, want)
        elif name == "Padding1":
            assert got.shape == (1, 1, 4, 4)
        else:
            check_asserts(asserts, {"output": got})
    elif suite == "TestConvolution1D":
        # tests/cpu/test-convolutions.cpp:11-126: convolve1D(input, kernel, stride, padding)
        stride, pad = {"Stride2": (2, 0), "Padding1": (1, 1)}.get(name, (1, 0))
        assert allclose(down(be.conv1d(up(t["input"]), up(t["kernel"]), stride, pad)), t["expected"])
    elif suite == "FunctionTests":
        # tests/cpu/test-functions.cpp:11-160: the expectation is the std:: function of each element
        fn = name.lower()
        x = t["A"]
        got = down(be.unary(fn, up(x), eps=1e-6))
        ref = {"log": math.log, "exp": math.exp, "sqrt": math.sqrt, "rsqrt": lambda v: 1.0 / math.sqrt(v + 1e-6), "abs": abs,
               "sin": math.sin, "cos": math.cos, "tan": math.tan, "sinh": math.sinh, "cosh": math.cosh, "tanh": math.tanh}[fn]
        want = torch.tensor([ref(float(v)) for v in x.flatten()], dtype=torch.float64).reshape(x.shape).float()
        assert allclose(got, want, rtol=1e-5, atol=1e-7)
    elif suite == "TestReductions":
        x = up(t["X"])
        named = {}
        if name == "Test1D":
            named = {"tmax": be.reduce("argmax", x, 0).reshape(1), "tmin": be.reduce("argmin", x, 0).reshape(1)}
        elif name == "Test2D":
            named = {"Zmax": be.reduce("argmax", x, -1), "Zmin": be.reduce("argmin", x, -1)}
        elif name == "Test2D_Axis0":
            named = {"Zmax": be.reduce("argmax", x, 0), "Zmin": be.reduce("argmin", x, 0)}
        elif name == "TestSum2D_Keepdim":
            named = {"result": be.reduce("sum", x, 1, True)}
            assert named["result"].shape == (2, 1)
        elif name == "TestMean2D":
            named = {"result": be.reduce("mean", x, 0)}
        elif name == "Test1D_MeanAndSum":
            named = {"tsum": be.reduce("sum", x, -1).reshape(1), "tmean": be.reduce("mean", x, -1).reshape(1)}
        elif name == "Test1D_MeanAndSum_Keepdim":
            named = {"tsum": be.reduce("sum", x, 0, True), "tmean": be.reduce("mean", x, 0, True)}
            assert named["tsum"].shape == (1,)
        elif name in ("Test2D_AxisMinus1_Keepdim", "Test3D_AxisMinus1_Keepdim"):
            named = {"tsum": be.reduce("sum", x, -1, True), "tmean": be.reduce("mean", x, -1, True)}
            assert named["tsum"].shape[-1] == 1
        elif name == "TestRMSIssued":  # mean(X*X, -1), test-reductions.cpp:162-175
            named = {"data": be.reduce("mean", be.binary("mul", x, x), -1).flatten()}
        check_asserts(asserts, {k: down(v) for k, v in named.items()})
    elif suite == "TransposedReshaped":
        # tests/cpu/test-non-contiguous.cpp:12-70: transpose(1,2) then reshape forces a repack of the view
        x = up(t["X"]).transpose(1, 2)
        got = down(be.unary("repack", x)).reshape(2, 4, 12)
        assert allclose(got, t["Y_expected"])
    else:
        pytest.skip("outside the path")


CASES = list(VECTORS)


@pytest.mark.parametrize("case", CASES)
def test_port_reproduces_reference_test(case):
    run_case(case, CpuBackend())


@pytest.mark.gpu
@pytest.mark.parametrize("case", CASES)
def test_cuda_path_reproduces_reference_test(case):
    run_case(case, GpuBackend())
