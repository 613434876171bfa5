"""Golden vectors produced by the reference's own CPU kernels (tests/golden/reference/*.tannic and
tests/golden/data_movement/*.tannic, one tensor per file in the reference's own `.tannic` record, made by
tests/golden/make_golden.py) for fp16 / bf16 / int32, which the reference's test-suite never
covers. CPU: the C restatement reproduces them bit for bit. GPU (marked): the CUDA path matches the
float-accumulating results within rtol 1e-2 / atol 1e-2, integers and indices exactly."""
from pathlib import Path

import pytest
import torch

import oracle
from tannic_b200 import serialization

GOLDEN = Path(__file__).parent / "golden"


def get(case, name):
    return serialization.load(GOLDEN / "reference" / f"{case}.{name}.tannic")


def same(a, b):
    return a.shape == b.shape and a.dtype == b.dtype and torch.equal(a.contiguous().view(torch.uint8), b.contiguous().view(torch.uint8))


def close(got, want, rtol=1e-2, atol=1e-2):
    g, w = got.double(), want.double()
    return got.shape == want.shape and bool(((g - w).abs() <= atol + rtol * w.abs()).all())


def expr(be_unary, be_binary, x, y):
    return be_binary("sub", be_binary("add", be_unary("log", x), be_binary("mul", y, y)), be_unary("exp", x))


def test_port_matches_golden_expression_and_add():
    for case in ("expr_fp16", "expr_bf16"):
        x, y = get(case, "x"), get(case, "y")
        got = expr(oracle.unary, oracle.binary, x, y)
        w = get(case, "z")
        # libm may differ from the build that made the fixture by an ulp of the storage type
        assert close(got, w, rtol=2 ** -7, atol=1e-3)
    assert same(oracle.binary("add", get("add_int32", "a"), get("add_int32", "b")), get("add_int32", "z"))


def test_port_matches_golden_gemm_conv_reductions():
    x, w = get("gemm_bf16", "x"), get("gemm_bf16", "w")
    assert same(oracle.matmul(x, w.t(), acc=oracle.ACC_STORAGE), get("gemm_bf16", "z"))
    assert same(oracle.matmul(x, w.t(), acc=oracle.ACC_WIDE), get("gemm_bf16", "z_wide"))
    q, k = get("scores_fp16", "q"), get("scores_fp16", "k")
    s = oracle.matmul(q, k.transpose(-1, -2), acc=oracle.ACC_WIDE)
    assert same(s, get("scores_fp16", "s_wide"))
    assert same(oracle.scale(s, 0.125), get("scores_fp16", "s_scaled"))
    xc, w3, w1, bias = (get("conv_fp16", n) for n in ("x", "w3", "w1", "bias"))
    assert same(oracle.conv2d(xc, w3, 1, 1, acc=oracle.ACC_STORAGE), get("conv_fp16", "y3"))
    assert same(oracle.conv2d(xc, w3, 1, 1, acc=oracle.ACC_WIDE), get("conv_fp16", "y3_wide"))
    assert same(oracle.conv2d(xc, w3, 1, 1, bias=bias, acc=oracle.ACC_WIDE), get("conv_fp16", "y3b_wide"))
    assert same(oracle.conv2d(xc, w1, 1, 0, acc=oracle.ACC_WIDE), get("conv_fp16", "y1_wide"))
    assert same(oracle.conv2d(xc, w3, 2, 1, acc=oracle.ACC_WIDE), get("conv_fp16", "y3s2_wide"))
    s = get("reduce_bf16", "s")
    assert same(oracle.reduce("argmax", s, -1), get("reduce_bf16", "argmax"))
    assert same(oracle.reduce("argmin", s, -1), get("reduce_bf16", "argmin"))
    assert same(oracle.reduce("argmax", s, 0), get("reduce_bf16", "argmax_axis0"))
    assert same(oracle.reduce("sum", s, -1, acc=oracle.ACC_STORAGE), get("reduce_bf16", "sum"))
    assert same(oracle.reduce("mean", s, -1, acc=oracle.ACC_STORAGE), get("reduce_bf16", "mean"))
    assert same(oracle.reduce("sum", s, -1, acc=oracle.ACC_WIDE), get("reduce_bf16", "sum_wide"))


@pytest.mark.gpu
def test_cuda_matches_golden():
    from tannic_b200 import _abi as A
    from tannic_b200 import ops as tb
    d = lambda t: t.cuda()  # noqa: E731
    for case in ("expr_fp16", "expr_bf16"):
        x, y = d(get(case, "x")), d(get(case, "y"))
        nodes = [(A.OP_LOG, 0, 0), (A.OP_MUL, 1, 1), (A.OP_ADD, 4, 5), (A.OP_EXP, 0, 0), (A.OP_SUB, 6, 7)]
        assert close(tb.program([x, y], nodes).cpu(), get(case, "z"))
        assert close(tb.sub(tb.add(tb.log(x), tb.mul(y, y)), tb.exp(x)).cpu(), get(case, "z"))
    assert same(tb.add(d(get("add_int32", "a")), d(get("add_int32", "b"))).cpu(), get("add_int32", "z"))
    x, w = d(get("gemm_bf16", "x")), d(get("gemm_bf16", "w"))
    assert close(tb.matmul(x, w.t()).cpu(), get("gemm_bf16", "z_wide"))
    q, k = d(get("scores_fp16", "q")), d(get("scores_fp16", "k"))
    assert close(tb.matmul(q, k.transpose(-1, -2)).cpu(), get("scores_fp16", "s_wide"))
    assert close(tb.matmul(q, k.transpose(-1, -2), scale_by=0.125).cpu(), get("scores_fp16", "s_scaled"))
    xc, w3, w1, bias = (d(get("conv_fp16", n)) for n in ("x", "w3", "w1", "bias"))
    assert close(tb.convolve2D(xc, w3, 1, 1).cpu(), get("conv_fp16", "y3_wide"))
    assert close(tb.convolve2D(xc, w3, 1, 1, bias=bias).cpu(), get("conv_fp16", "y3b_wide"))
    assert close(tb.convolve2D(xc, w1, 1, 0).cpu(), get("conv_fp16", "y1_wide"))
    assert close(tb.convolve2D(xc, w3, 2, 1).cpu(), get("conv_fp16", "y3s2_wide"))
    s = d(get("reduce_bf16", "s"))
    assert same(tb.argmax(s, -1).cpu(), get("reduce_bf16", "argmax"))
    assert same(tb.argmin(s, -1).cpu(), get("reduce_bf16", "argmin"))
    assert same(tb.argmax(s, 0).cpu(), get("reduce_bf16", "argmax_axis0"))
    assert close(tb.sum(s, -1).cpu(), get("reduce_bf16", "sum_wide"))
    mx, sm, am = tb.reduce_stats(s, -1)
    assert same(am.cpu(), get("reduce_bf16", "argmax")) and close(sm.cpu(), get("reduce_bf16", "sum_wide"))
    assert tb.device_errors() == 0


# ---- data movement around the path: tests/golden/data_movement (same generator script) ----

def mv(case, name):
    return serialization.load(GOLDEN / "data_movement" / f"{case}.{name}.tannic")


class _Port:
    def up(self, t): return t
    def down(self, t): return t
    repeat = staticmethod(lambda x, r, ax: oracle.repeat(x, r, ax))
    concat = staticmethod(lambda a, b, ax: oracle.concat(a, b, ax))
    triu = staticmethod(lambda x, k: oracle.triangular(x, True, k))
    tril = staticmethod(lambda x, k: oracle.triangular(x, False, k))
    outer = staticmethod(lambda a, b: oracle.outer(a, b))
    cartesian = staticmethod(lambda a, b: torch.view_as_real(oracle.complex_pair(a, b, False)))
    polar = staticmethod(lambda a, b: torch.view_as_real(oracle.complex_pair(a, b, True)))


class _Cuda:
    def __init__(self):
        from tannic_b200 import ops
        self.tb = ops

    def up(self, t): return t.cuda()
    def down(self, t): return t.cpu()
    def repeat(self, x, r, ax): return self.tb.repeat(x, r, ax)
    def concat(self, a, b, ax): return self.tb.concatenate(a, b, ax)
    def triu(self, x, k): return self.tb.triu(x, k)
    def tril(self, x, k): return self.tb.tril(x, k)
    def outer(self, a, b): return self.tb.outer(a, b)
    def cartesian(self, a, b): return torch.view_as_real(self.tb.cartesian(a, b))
    def polar(self, a, b): return torch.view_as_real(self.tb.polar(a, b))


def check_data_movement(be):
    u, dn = be.up, be.down
    x = u(mv("repeat_bf16", "x"))
    assert same(dn(be.repeat(x, 3, 1)), mv("repeat_bf16", "axis1_x3"))
    assert same(dn(be.repeat(x, 2, 0)), mv("repeat_bf16", "axis0_x2"))
    assert same(dn(be.repeat(x.transpose(0, 2), 2, 1)), mv("repeat_bf16", "permuted_axis1_x2"))
    a, b, c = (u(mv("concat", n)) for n in "abc")
    assert same(dn(be.concat(a, b, 1)), mv("concat", "ab_axis1"))
    assert same(dn(be.concat(a, c, 2)), mv("concat", "ac_axis2"))
    assert same(dn(be.concat(u(mv("concat", "m")), u(mv("concat", "n")), 0)), mv("concat", "mn_axis0"))
    f, i = u(mv("triangular", "f")), u(mv("triangular", "i"))
    assert same(dn(be.triu(f, 0)), mv("triangular", "f_triu0"))
    assert same(dn(be.tril(f, 1)), mv("triangular", "f_tril1"))
    assert same(dn(be.triu(i, 2)), mv("triangular", "i_triu2"))
    assert same(dn(be.tril(i, 0)), mv("triangular", "i_tril0"))
    assert same(dn(be.outer(u(mv("outer", "a")), u(mv("outer", "b")))), mv("outer", "ab"))
    assert same(dn(be.outer(u(mv("outer", "ia")), u(mv("outer", "ib")))), mv("outer", "iab"))
    rho, theta = u(mv("complex", "rho")), u(mv("complex", "theta"))
    assert same(dn(be.cartesian(rho, theta)), mv("complex", "cartesian"))
    assert close(dn(be.polar(rho, theta)), mv("complex", "polar"), rtol=1e-5, atol=1e-6)


def test_port_matches_golden_data_movement():
    check_data_movement(_Port())


@pytest.mark.gpu
def test_cuda_matches_golden_data_movement():
    check_data_movement(_Cuda())


# ---- conv1d and comparisons ----

def test_port_matches_golden_conv1d_and_comparisons():
    x, k = get("conv1d", "x"), get("conv1d", "k")
    assert same(oracle.conv1d(x, k, 2, 1, acc=oracle.ACC_STORAGE), get("conv1d", "y_s2p1"))
    assert same(oracle.conv1d(x, k, 2, 1, acc=oracle.ACC_WIDE), get("conv1d", "y_s2p1_wide"))
    assert same(oracle.conv1d(get("conv1d", "xi"), get("conv1d", "ki"), 1, 0), get("conv1d", "yi"))
    a, b = get("compare_bf16", "a"), get("compare_bf16", "b")
    for op in oracle.COMPARE:
        assert torch.equal(oracle.compare_packed(op, a, b)[0].view(torch.int8), get("compare_bf16", op))


@pytest.mark.gpu
def test_cuda_matches_golden_conv1d_and_comparisons():
    from tannic_b200 import ops as tb
    x, k = get("conv1d", "x").cuda(), get("conv1d", "k").cuda()
    assert close(tb.convolve1D(x, k, 2, 1).cpu(), get("conv1d", "y_s2p1_wide"))
    assert same(tb.convolve1D(get("conv1d", "xi").cuda(), get("conv1d", "ki").cuda(), 1, 0).cpu(), get("conv1d", "yi"))
    a, b = get("compare_bf16", "a").cuda(), get("compare_bf16", "b").cuda()
    for op in oracle.COMPARE:
        assert torch.equal(getattr(tb, op)(a, b).cpu().view(torch.int8), get("compare_bf16", op))
