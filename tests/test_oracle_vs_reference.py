"""Pins the C restatement (oracle/tannic_oracle.c) to the reference's own CPU kernels compiled
from its sources (oracle/_ref): bit-exact for integers, indices, half add/sub/mul and every
accumulation order; within 1 ulp of the storage type where libm is involved."""
import pytest
import torch

import oracle
from tannic_b200 import _abi as A

INTS = [torch.int8, torch.int16, torch.int32, torch.int64]
FLOATS = [torch.float16, torch.bfloat16, torch.float32, torch.float64]


def gen(shape, dtype, seed, lo=-4.0, hi=4.0):
    if dtype in INTS:
        return oracle.fill(shape, dtype, seed, "uniform", -100, 100)
    return oracle.fill(shape, dtype, seed, "uniform", lo, hi)


def same_bits(a, b):
    assert a.dtype == b.dtype and a.shape == b.shape
    ia = a.contiguous().view(torch.uint8) if a.dtype != torch.bool else a
    ib = b.contiguous().view(torch.uint8) if b.dtype != torch.bool else b
    return torch.equal(ia, ib)


def ulp_close(a, b, ulps=1):
    """|a-b| within `ulps` units in the last place of the storage type (NaN == NaN)."""
    if a.dtype in INTS:
        return torch.equal(a, b)
    eps = torch.finfo(a.dtype).eps
    x, y = a.double(), b.double()
    nan_ok = torch.isnan(x) == torch.isnan(y)
    x, y = torch.nan_to_num(x, nan=0.0), torch.nan_to_num(y, nan=0.0)
    inf = torch.isinf(x) | torch.isinf(y)
    ok = torch.where(inf, x == y, (x - y).abs() <= ulps * eps * torch.maximum(x.abs(), y.abs()) + 1e-300)
    return bool((ok & nan_ok).all())


@pytest.mark.parametrize("op", ["add", "sub", "mul"])
@pytest.mark.parametrize("da", INTS)
@pytest.mark.parametrize("db", INTS)
def test_int_pairs_bit_exact(ref_lib, op, da, db):
    a, b = gen((3, 1, 5), da, 1), gen((4, 5), db, 2)
    assert same_bits(oracle.binary(op, a, b), oracle.binary(op, a, b, impl="ref"))


@pytest.mark.parametrize("op", ["add", "sub", "mul", "pow"])
@pytest.mark.parametrize("pair", [
    (torch.float16, torch.float16), (torch.bfloat16, torch.bfloat16), (torch.float32, torch.float32),
    (torch.float64, torch.float64), (torch.float16, torch.float32), (torch.float32, torch.bfloat16),
    (torch.float16, torch.float64), (torch.float32, torch.float64), (torch.int32, torch.float32),
    (torch.float64, torch.int32),
])
def test_float_pairs(ref_lib, op, pair):
    da, db = pair
    lo, hi = (0.1, 3.0) if op == "pow" else (-4.0, 4.0)
    a = gen((2, 1, 7), da, 3, lo, hi) if da not in INTS else oracle.fill((2, 1, 7), da, 3, "uniform", 1, 4)
    b = gen((1, 5, 7), db, 4, lo, hi) if db not in INTS else oracle.fill((1, 5, 7), db, 4, "uniform", 1, 4)
    # The reference's pow(half, half) entry writes float32 into a half-sized result
    # (src/cpu/ops-binary.cpp:388): give it the float32 buffer it actually fills and compare values.
    out_dtype = None
    if op == "pow" and da == db and da in (torch.float16, torch.bfloat16):
        from tannic_b200 import _abi as A
        out_dtype = A.FLOAT32
    got = oracle.binary(op, a, b, out_dtype=out_dtype)
    want = oracle.binary(op, a, b, out_dtype=out_dtype, impl="ref")
    if op == "pow":
        assert ulp_close(got, want, 1)
    else:
        assert same_bits(got, want)


def test_strided_binary_operands(ref_lib):
    a = gen((6, 5), torch.float32, 5).t()       # [5, 6] view with strides (1, 5)
    b = gen((5, 12), torch.float32, 6)[:, ::2]  # [5, 6] view with strides (12, 2)
    assert same_bits(oracle.binary("add", a, b), oracle.binary("add", a, b, impl="ref"))


@pytest.mark.parametrize("name", ["neg", "repack", "log", "exp", "sqrt", "rsqrt", "abs", "sin", "cos", "tan", "sinh", "cosh", "tanh"])
@pytest.mark.parametrize("dtype", FLOATS)
def test_unary_floats(ref_lib, name, dtype):
    lo, hi = (0.1, 4.0) if name in ("log", "sqrt", "rsqrt") else (-3.0, 3.0)
    x = gen((3, 17), dtype, 7, lo, hi)
    got, want = oracle.unary(name, x, eps=1e-5), oracle.unary(name, x, eps=1e-5, impl="ref")
    if name in ("neg", "repack", "abs", "sqrt"):
        assert same_bits(got, want)
    else:
        assert ulp_close(got, want, 1)


@pytest.mark.parametrize("name,dtype", [("neg", torch.int8), ("neg", torch.int32), ("repack", torch.int16), ("abs", torch.int32), ("abs", torch.int64)])
def test_unary_ints(ref_lib, name, dtype):
    x = gen((4, 9), dtype, 8)
    assert same_bits(oracle.unary(name, x), oracle.unary(name, x, impl="ref"))


def test_unary_strided_source(ref_lib):
    x = gen((7, 4), torch.float32, 9, 0.1, 4.0).t()
    assert same_bits(oracle.unary("log", x), oracle.unary("log", x, impl="ref"))
    assert same_bits(oracle.unary("repack", x), oracle.unary("repack", x, impl="ref"))


@pytest.mark.parametrize("dtype", [torch.int32, torch.float16, torch.bfloat16, torch.float32, torch.float64])
def test_scale(ref_lib, dtype):
    x = gen((5, 6), dtype, 10)
    v = 3 if dtype in INTS else 0.125
    assert same_bits(oracle.scale(x, v), oracle.scale(x, v, impl="ref"))


@pytest.mark.parametrize("pair", [
    (torch.float32, torch.float32), (torch.float64, torch.float64), (torch.float16, torch.float16),
    (torch.bfloat16, torch.bfloat16), (torch.bfloat16, torch.float32), (torch.float16, torch.float32),
    (torch.int8, torch.int8), (torch.int32, torch.int32), (torch.int16, torch.int64), (torch.int32, torch.float32),
])
def test_gemm_literal(ref_lib, pair):
    """Storage-type accumulation, the literal behaviour of the reference CPU kernel."""
    da, db = pair
    a, b = gen((3, 9, 33), da, 11, -1, 1), gen((3, 33, 7), db, 12, -1, 1)
    got = oracle.matmul(a, b, acc=oracle.ACC_STORAGE)
    want = oracle.matmul(a, b, impl="ref")
    assert same_bits(got, want)


def test_gemm_transposed_and_broadcast(ref_lib):
    a = gen((2, 3, 6, 10), torch.float32, 13)
    w = gen((8, 10), torch.float32, 14)
    got = oracle.matmul(a, w.t(), acc=oracle.ACC_STORAGE)
    want = oracle.matmul(a, w.t(), impl="ref")
    assert same_bits(got, want)
    at = gen((10, 6), torch.float32, 15).t()
    assert same_bits(oracle.matmul(at, w.t(), acc=oracle.ACC_STORAGE), oracle.matmul(at, w.t(), impl="ref"))


def test_gemm_wide_accumulation_is_the_references_float_instantiation(ref_lib):
    """bf16 x bf16 with float32 accumulation == the reference's own <bhalf, float, float> kernel
    (src/cpu/matmul.cpp:228) run on the second operand up-converted exactly, rounded once."""
    a, b = gen((5, 200), torch.bfloat16, 16, -1, 1), gen((200, 4), torch.bfloat16, 17, -1, 1)
    want = oracle.matmul(a, b.float(), impl="ref").to(torch.bfloat16)
    got = oracle.matmul(a, b, acc=oracle.ACC_WIDE)
    assert same_bits(got, want)


def test_gemm_batch_counter_defect_is_reproducible(ref_lib):
    """The reference passes the batch counter through a uint8 (src/cpu/matmul.cpp:101): with 300
    batches, iterations 256..299 redo batches 0..43 and batches 256..299 are never written. The
    port reproduces that only when asked to; by default it computes all 300."""
    a, b = gen((300, 2, 3), torch.float32, 18), gen((300, 3, 2), torch.float32, 19)
    sentinel = 12345.0
    want = oracle.matmul(a, b, impl="ref", out=torch.full((300, 2, 2), sentinel))
    wrapped = oracle.matmul(a, b, acc=oracle.ACC_STORAGE, wrap_batch_u8=True, out=torch.full((300, 2, 2), sentinel))
    assert same_bits(wrapped, want)
    assert bool((want[256:] == sentinel).all())
    fixed = oracle.matmul(a, b, acc=oracle.ACC_STORAGE)
    assert same_bits(fixed[:256], want[:256])
    assert torch.allclose(fixed, torch.matmul(a, b), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16, torch.float64, torch.int32])
@pytest.mark.parametrize("stride,padding", [(1, 0), (1, 1), (2, 1), ((2, 1), (0, 2))])
def test_conv2d_literal(ref_lib, dtype, stride, padding):
    x, w = gen((2, 3, 7, 6), dtype, 20, -1, 1), gen((4, 3, 3, 2), dtype, 21, -1, 1)
    bias = gen((4,), dtype, 22, -1, 1)
    assert same_bits(oracle.conv2d(x, w, stride, padding, acc=oracle.ACC_STORAGE), oracle.conv2d(x, w, stride, padding, impl="ref"))
    assert same_bits(oracle.conv2d(x, w, stride, padding, bias=bias, acc=oracle.ACC_STORAGE),
                     oracle.conv2d(x, w, stride, padding, bias=bias, impl="ref"))


def test_conv2d_wide_is_the_references_float_instantiation(ref_lib):
    x, w = gen((1, 16, 6, 6), torch.float16, 23, -1, 1), gen((3, 16, 3, 3), torch.float16, 24, -1, 1)
    want = oracle.conv2d(x.float(), w.float(), 1, 1, impl="ref").to(torch.float16)
    assert same_bits(oracle.conv2d(x, w, 1, 1, acc=oracle.ACC_WIDE), want)


@pytest.mark.parametrize("kind", ["argmax", "argmin", "sum", "mean"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16, torch.float64, torch.int32, torch.int8])
@pytest.mark.parametrize("axis", [0, 1, -1])
def test_reductions_literal(ref_lib, kind, dtype, axis):
    if kind == "mean" and dtype in INTS:
        pytest.skip("mean is float-only in the reference")
    x = gen((4, 6, 5), dtype, 25)
    assert same_bits(oracle.reduce(kind, x, axis, acc=oracle.ACC_STORAGE), oracle.reduce(kind, x, axis, impl="ref"))
    xt = x.transpose(0, 2)
    assert same_bits(oracle.reduce(kind, xt, axis, acc=oracle.ACC_STORAGE), oracle.reduce(kind, xt, axis, impl="ref"))


def test_argmax_ties_nan_and_infinities(ref_lib):
    inf, nan = float("inf"), float("nan")
    x = torch.tensor([[1, 5, 5], [7, 7, 2], [-inf, -inf, -inf], [nan, -inf, 3], [nan, nan, nan], [nan, -inf, -inf]], dtype=torch.float32)
    for kind in ("argmax", "argmin"):
        got, want = oracle.reduce(kind, x, -1), oracle.reduce(kind, x, -1, impl="ref")
        assert torch.equal(got, want)
    assert oracle.reduce("argmax", x, -1).tolist() == [1, 0, 0, 2, 0, 0]


def test_sum_wide_is_the_references_float_path(ref_lib):
    x = gen((7, 197), torch.bfloat16, 26, -2, 2)
    want = oracle.reduce("sum", x.float(), -1, impl="ref").to(torch.bfloat16)
    assert same_bits(oracle.reduce("sum", x, -1, acc=oracle.ACC_WIDE), want)


# ---- data movement around the path -------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16, torch.float64, torch.int32, torch.int8, torch.int64])
@pytest.mark.parametrize("axis", [0, 1, 2])
def test_repeat_literal(ref_lib, dtype, axis):
    x = gen((3, 4, 5), dtype, 40)
    assert same_bits(oracle.repeat(x, 3, axis), oracle.repeat(x, 3, axis, impl="ref"))
    assert same_bits(oracle.repeat(x, 3, axis), torch.repeat_interleave(x, 3, axis))
    xt = x.transpose(0, 2)
    assert same_bits(oracle.repeat(xt, 2, axis), oracle.repeat(xt, 2, axis, impl="ref"))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int32, torch.float64])
def test_concat_literal_where_the_reference_is_right(ref_lib, dtype):
    """The reference walks the inner block with the stride of dimension axis + 1 only: exact for the
    last two axes, also on strided operands of rank 2."""
    a, b = gen((3, 4, 5), dtype, 41), gen((3, 2, 5), dtype, 42)
    assert same_bits(oracle.concat(a, b, 1), oracle.concat(a, b, 1, impl="ref"))
    c = gen((3, 4, 7), dtype, 43)
    assert same_bits(oracle.concat(a, c, 2), oracle.concat(a, c, 2, impl="ref"))
    m, n = gen((6, 4), dtype, 44), gen((5, 4), dtype, 45)
    assert same_bits(oracle.concat(m, n, 0), oracle.concat(m, n, 0, impl="ref"))
    assert same_bits(oracle.concat(m.t(), n.t(), 1), oracle.concat(m.t(), n.t(), 1, impl="ref"))
    assert same_bits(oracle.concat(a, b, 1), torch.cat([a, b], 1))


def test_concat_reference_defect_for_leading_axes(ref_lib):
    """Rank 3, axis 0: the reference multiplies the flat inner index by strides[1] and reads the wrong
    elements; the restatement (and the device path) concatenate."""
    a, b = gen((3, 4, 5), torch.float32, 46), gen((2, 4, 5), torch.float32, 47)
    assert torch.equal(oracle.concat(a, b, 0), torch.cat([a, b], 0))
    assert not torch.equal(oracle.concat(a, b, 0, impl="ref"), torch.cat([a, b], 0))


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16, torch.float64, torch.int32, torch.int64])
@pytest.mark.parametrize("k", [0, 1, 3])
def test_triangular_literal(ref_lib, dtype, k):
    m = gen((5, 7), dtype, 48)
    if dtype not in (torch.float16, torch.bfloat16):  # that translation unit of the reference is built without its half types
        for upper in (True, False):
            assert same_bits(oracle.triangular(m, upper, k), oracle.triangular(m, upper, k, impl="ref"))
            assert same_bits(oracle.triangular(m.t(), upper, k), oracle.triangular(m.t(), upper, k, impl="ref"))
    assert same_bits(oracle.triangular(m, True, k), torch.triu(m, k))
    assert same_bits(oracle.triangular(m, False, k), torch.tril(m, k))


def test_triangular_reference_defect_for_negative_diagonals(ref_lib):
    m = gen((5, 7), torch.float32, 49)
    assert torch.equal(oracle.triangular(m, True, -2), torch.triu(m, -2))
    assert torch.equal(oracle.triangular(m, False, -2), torch.tril(m, -2))
    assert not torch.equal(oracle.triangular(m, True, -2, impl="ref"), torch.triu(m, -2))


@pytest.mark.parametrize("pair", [(torch.float32, torch.float32), (torch.float64, torch.float64), (torch.float32, torch.float64),
                                  (torch.int32, torch.float32), (torch.int64, torch.int64)])
def test_outer_literal_where_the_table_type_is_the_promoted_one(ref_lib, pair):
    a, b = gen((6,), pair[0], 50), gen((9,), pair[1], 51)
    assert same_bits(oracle.outer(a, b), oracle.outer(a, b, impl="ref"))


def test_outer_reference_writes_wider_than_promoted(ref_lib):
    """(float16, float16) is a float32 kernel in the reference's table (src/cpu/outer.cpp:91) although the
    front-end allocates float16: read as float32 it equals the product rounded once."""
    a, b = gen((6,), torch.float16, 52, -2, 2), gen((9,), torch.float16, 53, -2, 2)
    wide = oracle.outer(a, b, out_dtype=A.FLOAT32, impl="ref")
    assert same_bits(oracle.outer(a, b), wide.to(torch.float16))


@pytest.mark.parametrize("pair", [(torch.float32, torch.float32), (torch.float64, torch.float64), (torch.float32, torch.float64)])
def test_complex_constructors(ref_lib, pair):
    rho, theta = gen((3, 1, 4), pair[0], 54, 0, 2), gen((1, 5, 4), pair[1], 55, -3, 3)
    assert same_bits(torch.view_as_real(oracle.complex_pair(rho, theta, False)), torch.view_as_real(oracle.complex_pair(rho, theta, False, impl="ref")))
    got, want = oracle.complex_pair(rho, theta, True), oracle.complex_pair(rho, theta, True, impl="ref")
    assert torch.allclose(torch.view_as_real(got), torch.view_as_real(want), rtol=1e-6, atol=1e-7)


@pytest.mark.parametrize("dtype", INTS + FLOATS)
@pytest.mark.parametrize("stride,pad", [(1, 0), (2, 1), (3, 2)])
def test_conv1d_bit_exact(ref_lib, dtype, stride, pad):
    """src/cpu/conv1d.cpp:16-127 against the H = 1 case of the conv2d restatement, storage-type accumulation."""
    x, w = gen((2, 3, 19), dtype, 40, -1, 1), gen((4, 3, 5), dtype, 41, -1, 1)
    if dtype in INTS:
        x, w = x % 5, w % 3
    got = oracle.conv1d(x, w, stride, pad, acc=oracle.ACC_STORAGE)
    want = oracle.conv1d(x, w, stride, pad, impl="ref")
    assert same_bits(got, want)
    # a strided signal (every second channel of a wider tensor)
    wide = gen((2, 6, 19), dtype, 42, -1, 1)
    if dtype in INTS:
        wide = wide % 5
    assert same_bits(oracle.conv1d(wide[:, ::2], w, stride, pad, acc=oracle.ACC_STORAGE), oracle.conv1d(wide[:, ::2], w, stride, pad, impl="ref"))


@pytest.mark.parametrize("dtype", INTS + FLOATS)
@pytest.mark.parametrize("op", list(oracle.COMPARE))
def test_comparisons_bit_exact(ref_lib, dtype, op):
    """src/cpu/cmps.cpp:16-204: bit-packed boolean results, including the padding bits of the last byte."""
    a, b = gen((3, 5, 7), dtype, 43), gen((3, 5, 7), dtype, 44)
    b[0], b[1, :2] = a[0], a[1, :2]          # equal runs
    if dtype not in INTS:
        a[2, 0, :3] = float("nan")
        b[2, 1, 0] = float("inf")
    got, _ = oracle.compare_packed(op, a, b)
    want, _ = oracle.compare_packed(op, a, b, impl="ref")
    assert torch.equal(got, want)
    # strided operands walk their own strides
    got, _ = oracle.compare_packed(op, a.transpose(0, 2), b.transpose(0, 2))
    want, _ = oracle.compare_packed(op, a.transpose(0, 2), b.transpose(0, 2), impl="ref")
    assert torch.equal(got, want)
    expect = {"eq": a == b, "ne": a != b, "gt": a > b, "ge": a >= b, "lt": a < b, "le": a <= b}[op]
    assert torch.equal(oracle.compare(op, a, b), expect)
