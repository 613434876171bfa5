"""Parity of the CUDA path (through the C ABI) against the oracle on seeded inputs.

Bit-exact for integer dtypes, index results and half add/sub/mul; rtol 1e-2 / atol 1e-2 for
fp16 / bf16; rtol 1e-4 (atol 1e-5 for sums that cancel) for fp32; 1e-12 for fp64.
"""
import pytest
import torch

import oracle
from tannic_b200 import _abi as A
from tannic_b200 import ops as tb

pytestmark = pytest.mark.gpu

INTS = [torch.int8, torch.int16, torch.int32, torch.int64]
HALVES = [torch.float16, torch.bfloat16]
FLOATS = HALVES + [torch.float32, torch.float64]
TOL = {torch.float16: (1e-2, 1e-2), torch.bfloat16: (1e-2, 1e-2), torch.float32: (1e-4, 1e-5), torch.float64: (1e-12, 1e-12)}


def dev(t):
    return t.cuda()


def gen(shape, dtype, seed, lo=-4.0, hi=4.0, kind="uniform"):
    if dtype in INTS:
        return oracle.fill(shape, dtype, seed, "uniform", -100, 100)
    return oracle.fill(shape, dtype, seed, kind, lo, hi)


def assert_same(got, want):
    got = got.cpu()
    assert got.dtype == want.dtype and got.shape == want.shape
    if got.dtype in INTS:
        assert torch.equal(got, want)
    else:
        assert torch.equal(got.contiguous().view(torch.int16 if got.element_size() == 2 else torch.int32 if got.element_size() == 4 else torch.int64),
                           want.contiguous().view(torch.int16 if want.element_size() == 2 else torch.int32 if want.element_size() == 4 else torch.int64))


def assert_close(got, want, tol=None):
    got = got.cpu()
    assert got.dtype == want.dtype and got.shape == want.shape, (got.dtype, want.dtype, got.shape, want.shape)
    if got.dtype in INTS:
        assert torch.equal(got, want)
        return
    rtol, atol = tol or TOL[got.dtype]
    g, w = got.double(), want.double()
    bad = ~(((g - w).abs() <= atol + rtol * w.abs()) | (torch.isnan(g) & torch.isnan(w)) | ((g == w)))
    assert not bool(bad.any()), f"{int(bad.sum())} of {bad.numel()} outside tolerance; max abs diff {float((g - w).abs()[~torch.isnan(g - w)].max())}"


# ---------------------------------------------------------------- elementwise ----------

@pytest.mark.parametrize("op", ["add", "sub", "mul"])
@pytest.mark.parametrize("dtype", INTS + FLOATS)
@pytest.mark.parametrize("shapes", [((64, 96), (64, 96)), ((33, 64), (1, 64)), ((33, 64), (33, 1)), ((2, 1, 3), (1, 4, 3)),
                                    ((5, 7), (7,)), ((1000,), (1,)), ((), ()), ((3, 197), (3, 197))])
def test_binary_same_dtype_exact(op, dtype, shapes):
    a, b = gen(shapes[0], dtype, 1), gen(shapes[1], dtype, 2)
    want = oracle.binary(op, a, b)
    got = getattr(tb, op)(dev(a), dev(b))
    assert_same(got, want)


@pytest.mark.parametrize("dtype", FLOATS)
def test_pow(dtype):
    a, b = gen((40, 64), dtype, 3, 0.1, 3.0), gen((1, 64), dtype, 4, -2.0, 2.0)
    assert_close(tb.pow(dev(a), dev(b)), oracle.binary("pow", a, b))


@pytest.mark.parametrize("pair", [(torch.float16, torch.float32), (torch.float32, torch.bfloat16), (torch.float16, torch.float64),
                                  (torch.int32, torch.float32), (torch.float64, torch.int32), (torch.int8, torch.int32),
                                  (torch.int64, torch.int16), (torch.float32, torch.float64)])
@pytest.mark.parametrize("op", ["add", "mul", "sub"])
def test_binary_mixed_dtypes(pair, op):
    a, b = gen((9, 1, 11), pair[0], 5), gen((6, 11), pair[1], 6)
    want = oracle.binary(op, a, b)
    got = getattr(tb, op)(dev(a), dev(b))
    if want.dtype in INTS:
        assert_same(got, want)
    else:
        assert_close(got, want)


@pytest.mark.parametrize("pair", [(torch.float16, torch.float32), (torch.float32, torch.float16), (torch.bfloat16, torch.float32),
                                  (torch.float32, torch.bfloat16), (torch.float32, torch.float64), (torch.float64, torch.float32),
                                  (torch.int32, torch.float32), (torch.float32, torch.int32)])
@pytest.mark.parametrize("op", ["add", "sub", "mul", "pow"])
def test_binary_mixed_dtypes_dense_vector_path(pair, op):
    """Dense operands of two types take the eight-elements-per-thread kernel from 4096 elements on; a length
    that is not a multiple of eight exercises its tail. Same arithmetic as the element-wise kernel."""
    lo, hi = (0.1, 3.0) if op == "pow" else (-4.0, 4.0)
    a, b = gen((37, 333), pair[0], 5, lo, hi), gen((37, 333), pair[1], 6, lo, hi)
    if op == "pow" and torch.int32 in pair:
        a, b = a.abs() + 1, (b.abs() % 3) + 1
    want = oracle.binary(op, a, b)
    got = getattr(tb, op)(dev(a), dev(b))
    assert got.dtype == want.dtype
    if op == "pow":
        assert_close(got, want, tol=(1e-4, 1e-4) if want.dtype == torch.float32 else None)
    else:
        assert_same(got, want)


def test_binary_half_with_int_writes_result_dtype():
    """The reference's (float16, int32) entry writes float32 into a float16-sized buffer
    (src/cpu/ops-binary.cpp:199-206); the device path writes exactly dst->dtype."""
    a, b = gen((8, 8), torch.float16, 7), oracle.fill((8, 8), torch.int32, 8, "uniform", -20, 20)
    got = tb.add(dev(a), dev(b))
    assert got.dtype == torch.float16
    assert_close(got, (a.float() + b.float()).to(torch.float16))


@pytest.mark.parametrize("pair", [(torch.float16, torch.bfloat16), (torch.float32, torch.int8), (torch.float64, torch.int64)])
def test_binary_unsupported_pairs(pair):
    a, b = gen((4,), pair[0], 9), gen((4,), pair[1], 10)
    with pytest.raises(A.TannicError) as e:
        tb.add(dev(a), dev(b))
    assert e.value.status == A.UNSUPPORTED_DTYPE
    with pytest.raises(A.TannicError) as e:
        tb.pow(dev(gen((4,), torch.int32, 1)), dev(gen((4,), torch.int32, 2)))
    assert e.value.status == A.UNSUPPORTED_DTYPE


def test_binary_strided_views():
    a0, b0 = gen((48, 40), torch.float32, 11), gen((40, 96), torch.float32, 12)
    want = oracle.binary("add", a0.t(), b0[:, ::2])
    assert_same(tb.add(dev(a0).t(), dev(b0)[:, ::2]), want)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32, torch.int32])
def test_large_operations_on_strided_views(dtype):
    """Above 2^20 elements a transposed / permuted / sliced operand is copied dense first and the vector kernel
    runs; results stay bit-identical to the element-by-element evaluation of the same views."""
    a, b = gen((1100, 1000), dtype, 22), gen((1000, 1100), dtype, 23)
    assert_same(tb.add(dev(a), dev(b).t()), oracle.binary("add", a, b.t()))
    assert_same(tb.mul(dev(a).t(), dev(b)), oracle.binary("mul", a.t(), b))
    c = gen((1100, 2000), dtype, 24)
    assert_same(tb.sub(dev(c)[:, ::2], dev(a)), oracle.binary("sub", c[:, ::2], a))
    x4, y4 = gen((6, 12, 197, 80), dtype, 25), gen((6, 197, 12, 80), dtype, 26)
    assert_same(tb.add(dev(x4), dev(y4).permute(0, 2, 1, 3)), oracle.binary("add", x4, y4.permute(0, 2, 1, 3)))
    if dtype != torch.int32:
        p = gen((1100, 1000), dtype, 27, 0.1, 4.0)
        assert_close(tb.log(dev(p).t()), oracle.unary("log", p.t()))
        assert_same(tb.neg(dev(p).t()), oracle.unary("neg", p.t()))
    # a broadcast operand next to a strided one keeps its broadcast
    row = gen((1, 1000), dtype, 28)
    assert_same(tb.add(dev(b).t(), dev(row)), oracle.binary("add", b.t(), row))


@pytest.mark.parametrize("name", ["neg", "repack", "log", "exp", "sqrt", "rsqrt", "abs", "sin", "cos", "tan", "sinh", "cosh", "tanh"])
@pytest.mark.parametrize("dtype", FLOATS)
@pytest.mark.parametrize("shape", [(64, 128), (3, 197), (1,), ()])
def test_unary(name, dtype, shape):
    lo, hi = (0.1, 4.0) if name in ("log", "sqrt", "rsqrt") else (-3.0, 3.0)
    x = gen(shape, dtype, 13, lo, hi)
    want = oracle.unary(name, x, eps=1e-5)
    got = tb.rsqrt(dev(x), 1e-5) if name == "rsqrt" else getattr(tb, name)(dev(x))
    if name in ("neg", "repack", "abs"):
        assert_same(got, want)
    else:
        assert_close(got, want)


@pytest.mark.parametrize("name,dtype", [("neg", torch.int8), ("neg", torch.int64), ("repack", torch.int16), ("abs", torch.int32), ("abs", torch.int64)])
def test_unary_ints(name, dtype):
    x = gen((17, 33), dtype, 14)
    assert_same(getattr(tb, name)(dev(x)), oracle.unary(name, x))


def test_unary_rejects_integer_log():
    with pytest.raises(A.TannicError) as e:
        tb.log(dev(gen((4,), torch.int32, 1)))
    assert e.value.status == A.UNSUPPORTED_DTYPE


def test_unary_strided_source():
    x = gen((70, 40), torch.float16, 15, 0.1, 4.0)
    assert_close(tb.log(dev(x).t()), oracle.unary("log", x.t()))
    assert_same(tb.repack(dev(x).t()), oracle.unary("repack", x.t()))
    assert_same(tb.repack(dev(x)[::2, 1::3]), oracle.unary("repack", x[::2, 1::3]))


@pytest.mark.parametrize("dtype", [torch.int8, torch.float16, torch.bfloat16, torch.float32, torch.float64, torch.int64])
@pytest.mark.parametrize("shape,perm", [((70, 45), (1, 0)), ((3, 197, 12, 64), (0, 2, 1, 3)), ((5, 33, 100), (0, 2, 1)), ((4, 50, 6, 40), (3, 1, 2, 0)),
                                        ((2, 3, 64, 96), (0, 1, 3, 2)), ((17, 16), (1, 0)), ((2, 1, 300, 20), (3, 0, 1, 2))])
def test_repack_of_permuted_views(dtype, shape, perm):
    """Views that permute dimensions: runs that stay contiguous move as 16-byte words, transposing views go
    through 32 x 32 shared-memory tiles, everything else element by element; all bit-exact."""
    x = gen(shape, dtype, 21)
    v = x.permute(*perm)
    assert_same(tb.repack(dev(x).permute(*perm)), v.contiguous())
    assert_same(tb.repack(dev(x).permute(*perm)), oracle.unary("repack", v))
    out = torch.empty(v.shape, dtype=dtype, device="cuda")
    tb.cpy(dev(x).permute(*perm), out)
    assert_same(out, v.contiguous())
    sliced = dev(x).permute(*perm)[..., 1::2]
    assert_same(tb.repack(sliced), v[..., 1::2].contiguous())


@pytest.mark.parametrize("dtype,value", [(torch.int32, 3), (torch.int8, -7), (torch.float16, 0.125), (torch.bfloat16, 0.125), (torch.float32, 1.7), (torch.float64, -2.5)])
def test_scale(dtype, value):
    x = gen((31, 64), dtype, 16)
    assert_same(tb.scale(dev(x), value), oracle.scale(x, value))


def _program_oracle(x, y):
    t0 = oracle.unary("log", x)
    t1 = oracle.binary("mul", y, y)
    t2 = oracle.binary("add", t0, t1)
    t3 = oracle.unary("exp", x)
    return oracle.binary("sub", t2, t3)


CFG2_NODES = [(A.OP_LOG, 0, 0), (A.OP_MUL, 1, 1), (A.OP_ADD, 4, 5), (A.OP_EXP, 0, 0), (A.OP_SUB, 6, 7)]


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shapes", [((96, 256), (1, 256)), ((96, 256), (96, 256)), ((96, 256), (96, 1)), ((5, 197), (1, 197)), ((4, 3, 8), (3, 1))])
def test_fused_program_matches_node_chain(dtype, shapes):
    """Z = log(X) + Y*Y - exp(X) in one kernel == the reference's five-node chain, node by node
    rounded to the storage dtype."""
    x, y = gen(shapes[0], dtype, 17, 0.1, 4.0), gen(shapes[1], dtype, 18, -2.0, 2.0)
    got = tb.program([dev(x), dev(y)], CFG2_NODES)
    assert_close(got, _program_oracle(x, y))
    # and the unfused device chain agrees with the same oracle
    dx, dy = dev(x), dev(y)
    chain = tb.sub(tb.add(tb.log(dx), tb.mul(dy, dy)), tb.exp(dx))
    assert_close(chain, _program_oracle(x, y))


@pytest.mark.parametrize("shapes", [((1000, 256), (1, 256)), ((37, 64), (37, 64)), ((5, 8), (5, 1)), ((64,), (64,))])
@pytest.mark.parametrize("pinned", ["near", "torch", "pageable"])
def test_host_program_matches_device_call(shapes, pinned):
    """Host buffers in and out through the library's chunked three-stream path (tn_eltwise_program_host)
    == the device call on resident tensors, bit for bit; two calls in a row reuse the staging memory.
    Pinned memory from the backend's own allocator, from torch, and pageable memory all give the same."""
    x, y = gen(shapes[0], torch.float16, 19, 0.1, 4.0), gen(shapes[1], torch.float16, 20, -2.0, 2.0)
    want = tb.program([dev(x), dev(y)], CFG2_NODES).cpu()
    keep = []
    if pinned == "near":
        bx, by, bo = tb.PinnedBuffer(x.shape, x.dtype), tb.PinnedBuffer(y.shape, y.dtype), tb.PinnedBuffer(want.shape, want.dtype)
        bx.tensor.copy_(x)
        by.tensor.copy_(y)
        keep = [bx, by, bo]
        hx, hy, out = bx.tensor, by.tensor, bo.tensor
    elif pinned == "torch":
        hx, hy, out = x.pin_memory(), y.pin_memory(), torch.empty(want.shape, dtype=torch.float16).pin_memory()
    else:
        hx, hy, out = x, y, torch.empty(want.shape, dtype=torch.float16)
    for chunks in (0, 3):
        out.zero_()
        tb.program_host([hx, hy], CFG2_NODES, out, chunks=chunks)
        assert_same(out.clone(), want)
    assert_close(out.clone(), _program_oracle(x, y))
    del keep


def test_host_program_refuses_device_and_strided_tensors():
    x = gen((8, 16), torch.float16, 19, 0.1, 4.0)
    out = torch.empty((8, 16), dtype=torch.float16)
    with pytest.raises(A.TannicError):
        tb.program_host([dev(x), x], CFG2_NODES, out)
    with pytest.raises(A.TannicError):
        tb.program_host([x.t(), x.t()], CFG2_NODES, torch.empty((16, 8), dtype=torch.float16))
    assert isinstance(tb.numa_node(0), int)


@pytest.mark.parametrize("dtype", HALVES)
@pytest.mark.parametrize("batches,m,n,k,scale", [(5, 197, 197, 64, 0.125), (3, 300, 250, 128, None), (7, 33, 7, 64, 0.5), (2, 128, 256, 192, 2.0),
                                                 (1, 5, 1, 8, None), (4, 130, 64, 64, 0.25), (2, 100, 300, 64, 0.5)])
def test_matmul_with_fused_row_statistics(dtype, batches, m, n, k, scale):
    """tn_gemm_scaled_stats: the product, and max / sum / argmax of each of its rows from the same kernel.
    S must equal what tn_gemm_scaled writes, bit for bit; argmax and max must be exactly those of that S
    (the oracle's reduction applied to it), the sum within the 16-bit tolerance. The last shape (300
    columns) is wider than one tile and takes the product followed by one reduction pass."""
    a, w = gen((batches, m, k), dtype, 64, -1, 1), gen((batches, n, k), dtype, 65, -1, 1)
    da, dw = dev(a), dev(w).transpose(-1, -2)
    plain = tb.matmul(da, dw, scale_by=scale)
    s, mx, sm, am = tb.matmul_stats(da, dw, scale_by=scale)
    assert_same(s, plain.cpu())
    host = s.cpu()
    assert torch.equal(am.cpu(), oracle.reduce("argmax", host, -1))
    assert_same(mx, oracle.reduce("max", host, -1))
    assert_close(sm, oracle.reduce("sum", host, -1, acc=oracle.ACC_WIDE))
    want = oracle.matmul(a[0], w[0].t(), acc=oracle.ACC_WIDE)
    assert_close(s[0], oracle.scale(want, scale) if scale is not None else want)
    assert tb.device_errors() == 0


def test_matmul_fused_statistics_ties_nan_and_infinities():
    """Rows built so that the maximum repeats (first occurrence wins, across even/odd columns and across
    32-column chunks), is -inf everywhere (index 0), or sits beside NaNs (never selected)."""
    n, k = 197, 64
    # batch b: A_b = e_0 (one row), W_b[:, 0] = the wanted row, other columns zero -> S_b[0, j] = W_b[j, 0]
    rows = torch.full((8, n), -1.0)
    rows[0, :] = 1.0                                          # every column equal: 0
    rows[1, [5, 69, 133]] = 3.0                               # ties in three chunks: 5
    rows[2, [63, 0]] = 2.0                                    # an odd and an even column tie: 0
    rows[3, :] = float("-inf")                                # all -inf: index 0
    rows[4, :] = float("nan"); rows[4, [40, 104]] = -5.0      # NaN is never selected: 40
    rows[5, [33, 1]] = 7.0                                    # odd columns in two chunks: 1
    rows[6, [62, 63]] = 1.5                                   # neighbours in one pair: 62
    rows[7, [196, 4]] = 0.0                                   # the last column of the ragged chunk and 4: 4
    w = torch.zeros((8, n, k), dtype=torch.bfloat16)
    w[:, :, 0] = rows.to(torch.bfloat16)
    a = torch.zeros((8, 1, k), dtype=torch.bfloat16)
    a[:, 0, 0] = 1.0
    s, mx, sm, am = tb.matmul_stats(dev(a), dev(w).transpose(-1, -2))
    host = s.cpu()
    assert torch.equal(am.cpu(), oracle.reduce("argmax", host, -1))
    assert am.cpu().flatten().tolist() == [0, 5, 0, 0, 40, 1, 62, 4]
    assert_same(mx, oracle.reduce("max", host, -1))


def test_fused_program_dynamic_and_other_static_shapes():
    x, w, b = gen((64, 128), torch.float32, 19), gen((64, 128), torch.float32, 20), gen((128,), torch.float32, 21)
    want = oracle.binary("add", oracle.binary("mul", x, w), b)
    assert_same(tb.program([dev(x), dev(w), dev(b)], [(A.OP_MUL, 0, 1), (A.OP_ADD, 4, 2)]), want)
    # a program that is not in the compiled set runs on the interpreter
    want = oracle.unary("tanh", oracle.binary("sub", oracle.unary("abs", x), w))
    got = tb.program([dev(x), dev(w)], [(A.OP_ABS, 0, 0), (A.OP_SUB, 4, 1), (A.OP_TANH, 5, 5)])
    assert_close(got, want)
    got = tb.program([dev(x), dev(w)], [(A.OP_SCALE, 0, 0, 0.5), (A.OP_RSQRT, 1, 1, 9.0), (A.OP_MUL, 4, 5)])
    want = oracle.binary("mul", oracle.scale(x, 0.5), oracle.unary("rsqrt", w, eps=9.0))
    assert_close(got, want)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_program_in_any_node_order_takes_the_compiled_form(dtype):
    """The same expression with its nodes listed in another order, the operands of an add / multiply
    swapped and the inputs numbered the other way round is rewritten into the compiled program: the
    result is bit-identical to the canonical listing (and so to the node-by-node chain)."""
    x, y = gen((300, 512), dtype, 90, 0.1, 4.0), gen((1, 512), dtype, 91, -2.0, 2.0)
    dx, dy = dev(x), dev(y)
    canonical = tb.program([dx, dy], CFG2_NODES)
    # exp first, operands of the add swapped
    reordered = [(A.OP_EXP, 0, 0), (A.OP_LOG, 0, 0), (A.OP_MUL, 1, 1), (A.OP_ADD, 6, 5), (A.OP_SUB, 7, 4)]
    assert_same(tb.program([dx, dy], reordered), canonical.cpu())
    # inputs the other way round: Y is input 0, X input 1
    renumbered = [(A.OP_MUL, 0, 0), (A.OP_LOG, 1, 1), (A.OP_EXP, 1, 1), (A.OP_ADD, 5, 4), (A.OP_SUB, 7, 6)]
    assert_same(tb.program([dy, dx], renumbered), canonical.cpu())
    # x0*x1 + x2 written as x2 + x1*x0
    a, b, c = dev(gen((64, 256), dtype, 92)), dev(gen((64, 256), dtype, 93)), dev(gen((256,), dtype, 94))
    want = tb.program([a, b, c], [(A.OP_MUL, 0, 1), (A.OP_ADD, 4, 2)])
    assert_same(tb.program([c, b, a], [(A.OP_MUL, 1, 2), (A.OP_ADD, 0, 4)]), want.cpu())
    # a different expression of the same size must not be mistaken for it: log(x) + y*y - exp(y)
    other = [(A.OP_LOG, 0, 0), (A.OP_MUL, 1, 1), (A.OP_ADD, 4, 5), (A.OP_EXP, 1, 1), (A.OP_SUB, 6, 7)]
    wide_y = dev(gen((300, 512), dtype, 95, -2.0, 2.0))
    got = tb.program([dx, wide_y], other)
    chain = tb.sub(tb.add(tb.log(dx), tb.mul(wide_y, wide_y)), tb.exp(wide_y))
    assert_close(got, chain.cpu())


@pytest.mark.parametrize("dtype", HALVES)
def test_interpreted_programs_of_many_shapes(dtype):
    """16-bit expressions outside the compiled set (the in-kernel interpreter): trees of several depths,
    `x op x`, a subtree used twice, non-commutative operand order, immediates, a column-broadcast input
    and a five-deep right-leaning chain: all against the oracle's node-by-node chain; the exact
    operations also bit for bit against the device's own node-by-node chain."""
    x, w = gen((130, 264), dtype, 100, 0.2, 3.0), gen((130, 264), dtype, 101, -2.0, 2.0)
    b, col = gen((264,), dtype, 102, -1.0, 1.0), gen((130, 1), dtype, 103, 0.5, 1.5)
    dx, dw, db, dcol = dev(x), dev(w), dev(b), dev(col)
    O, B, U = oracle, oracle.binary, oracle.unary
    # tanh(x*w + b) * 0.5 - rsqrt(x, 1e-3)
    got = tb.program([dx, dw, db], [(A.OP_MUL, 0, 1), (A.OP_ADD, 4, 2), (A.OP_TANH, 5, 5), (A.OP_SCALE, 6, 6, 0.5), (A.OP_RSQRT, 0, 0, 1e-3), (A.OP_SUB, 7, 8)])
    want = B("sub", O.scale(U("tanh", B("add", B("mul", x, w), b)), 0.5), U("rsqrt", x, eps=1e-3))
    assert_close(got, want)
    # exact operations only: ((x - w) * (x - w) + |w|) * col - x, with (x - w) written once and used twice
    nodes = [(A.OP_SUB, 0, 1), (A.OP_MUL, 4, 4), (A.OP_ABS, 1, 1), (A.OP_ADD, 5, 6), (A.OP_MUL, 7, 2), (A.OP_SUB, 8, 0)]
    got = tb.program([dx, dw, dcol], nodes)
    d_ = tb.sub(dx, dw)
    chain = tb.sub(tb.mul(tb.add(tb.mul(d_, d_), tb.abs(dw)), dcol), dx)
    assert_same(got, chain.cpu())
    diff = B("sub", x, w)
    assert_same(got, B("sub", B("mul", B("add", B("mul", diff, diff), U("abs", w)), col), x))
    # operand order of the non-commutative ones: w - (x - b), pow(x, w)
    got = tb.program([dx, dw, db], [(A.OP_SUB, 0, 2), (A.OP_SUB, 1, 4)])
    assert_same(got, B("sub", w, B("sub", x, b)))
    got = tb.program([dx, dw], [(A.OP_POW, 0, 1), (A.OP_NEG, 4, 4), (A.OP_EXP, 5, 5)])
    assert_close(got, U("exp", U("neg", B("pow", x, w))))
    # the same value feeding two different nodes (evaluated twice on the stack): (x+w) * (x+w - b)
    got = tb.program([dx, dw, db], [(A.OP_ADD, 0, 1), (A.OP_SUB, 4, 2), (A.OP_MUL, 4, 5)])
    sm_ = B("add", x, w)
    assert_same(got, B("mul", sm_, B("sub", sm_, b)))
    # a right-leaning chain of subtractions five deep: x - (w - (x - (w - (x - b))))
    nodes = [(A.OP_SUB, 0, 2), (A.OP_SUB, 1, 4), (A.OP_SUB, 0, 5), (A.OP_SUB, 1, 6), (A.OP_SUB, 0, 7)]
    got = tb.program([dx, dw, db], nodes)
    assert_same(got, B("sub", x, B("sub", w, B("sub", x, B("sub", w, B("sub", x, b))))))


def test_fused_program_rejects_bad_programs():
    x = dev(gen((8,), torch.float32, 1))
    with pytest.raises(A.TannicError):
        tb.program([x], [(A.OP_ADD, 0, 5)])  # reads a value defined later
    with pytest.raises(A.TannicError):
        tb.program([x], [(99, 0, 0)])


# ---------------------------------------------------------------- reductions -----------

@pytest.mark.parametrize("kind", ["argmax", "argmin", "sum", "mean", "max"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16, torch.float64, torch.int32, torch.int8])
@pytest.mark.parametrize("shape,axis", [((6, 197), -1), ((33, 7, 5), 1), ((33, 7, 5), 0), ((4, 3, 9000), -1), ((5, 64), -1), ((7,), 0), ((3, 1, 4), 1)])
def test_reductions(kind, dtype, shape, axis):
    if kind == "mean" and dtype in INTS:
        pytest.skip("mean is float-only in the reference")
    x = gen(shape, dtype, 22, -2.0, 2.0)
    want = oracle.reduce(kind, x, axis, acc=oracle.ACC_WIDE)
    got = getattr(tb, kind)(dev(x), axis)
    if kind in ("argmax", "argmin", "max") or dtype in INTS:
        assert_same(got, want)
    else:
        assert_close(got, want)


@pytest.mark.parametrize("kind", ["argmax", "sum", "argmin"])
def test_reductions_strided_views(kind):
    x = gen((12, 9, 10), torch.float32, 23)
    for view in (lambda t: t.transpose(0, 2), lambda t: t[:, ::2, 1:], lambda t: t.permute(1, 2, 0)):
        for axis in (0, 1, 2):
            want = oracle.reduce(kind, view(x), axis, acc=oracle.ACC_WIDE)
            got = getattr(tb, kind)(view(dev(x)), axis)
            if kind == "sum":
                assert_close(got, want)
            else:
                assert_same(got, want)


def test_argmax_ties_nan_infinities():
    inf, nan = float("inf"), float("nan")
    rows = [[1, 5, 5], [7, 7, 2], [-inf, -inf, -inf], [nan, -inf, 3], [nan, nan, nan], [nan, -inf, -inf], [inf, inf, 1]]
    for dtype in (torch.float32, torch.float16, torch.bfloat16):
        x = torch.tensor(rows, dtype=dtype)
        assert tb.argmax(dev(x), -1).cpu().tolist() == oracle.reduce("argmax", x, -1).tolist() == [1, 0, 0, 2, 0, 0, 0]
        assert tb.argmin(dev(x), -1).cpu().tolist() == oracle.reduce("argmin", x, -1).tolist()
        assert tb.argmax(dev(x), 0).cpu().tolist() == oracle.reduce("argmax", x, 0).tolist()
    # long rows with the maximum repeated across lanes / segments
    x = torch.zeros(3, 5000, dtype=torch.bfloat16)
    x[0, 4999] = 1
    x[0, 77] = 1
    x[1, 4096] = 2
    x[1, 4097] = 2
    assert tb.argmax(dev(x), -1).cpu().tolist() == [77, 4096, 0]


def test_reduce_keepdim_and_stats():
    x = gen((8, 12, 197), torch.bfloat16, 24, -2.0, 2.0)
    assert tb.sum(dev(x), -1, keepdim=True).shape == (8, 12, 1)
    mx, sm, am = tb.reduce_stats(dev(x), -1)
    assert_same(am, oracle.reduce("argmax", x, -1))
    assert_same(mx, oracle.reduce("max", x, -1))
    assert_close(sm, oracle.reduce("sum", x, -1, acc=oracle.ACC_WIDE))


@pytest.mark.parametrize("dtype", HALVES)
@pytest.mark.parametrize("shape", [(4100, 197), (5000, 9), (4113, 400), (6000, 64), (4500, 33), (21, 12, 197, 197), (4097, 8), (4200, 255)])
def test_reductions_one_thread_per_row(dtype, shape):
    """Many short 16-bit rows take the kernel in which a warp stages a span of 32 rows and every lane
    reduces one of them: even and odd row lengths (rows that start in either half of a word), a row count
    that is not a multiple of 32, coarse values (many ties: the first occurrence must win), rows with NaN,
    infinities and all -inf; every reduction kind and the fused statistics, against the oracle."""
    x = gen(shape, dtype, 61, -2.0, 2.0)
    flat = x.view(-1, shape[-1])
    flat[1::3] = (flat[1::3] * 4).round() / 4          # ties
    flat[2, :] = float("-inf")
    flat[3, :] = float("nan")
    flat[4, 1::2] = float("nan")
    flat[5, 3] = float("inf")
    flat[5, 6] = float("inf")
    flat[6, :] = 0.0
    flat[6, 5] = -0.0
    dx = dev(x)
    for kind in ("argmax", "argmin", "max"):
        assert_same(getattr(tb, kind)(dx, -1), oracle.reduce(kind, x, -1))
    ok_rows = torch.ones(flat.shape[0], dtype=torch.bool)
    ok_rows[[2, 3, 4, 5]] = False                       # sums of rows with NaN / inf are not compared
    want_sum = oracle.reduce("sum", x, -1, acc=oracle.ACC_WIDE).reshape(-1)[ok_rows]
    assert_close(tb.sum(dx, -1).reshape(-1)[dev(ok_rows)], want_sum)
    assert_close(tb.mean(dx, -1).reshape(-1)[dev(ok_rows)], oracle.reduce("mean", x, -1, acc=oracle.ACC_WIDE).reshape(-1)[ok_rows])
    mx, sm, am = tb.reduce_stats(dx, -1)
    assert_same(am, oracle.reduce("argmax", x, -1))
    assert_same(mx, oracle.reduce("max", x, -1))
    assert_close(sm.reshape(-1)[dev(ok_rows)], want_sum)


@pytest.mark.parametrize("dtype,shape", [(torch.bfloat16, (12, 197, 197)), (torch.float16, (4099, 64)), (torch.float32, (3001, 100)),
                                         (torch.int32, (2500, 33)), (torch.float64, (2100, 8)), (torch.int8, (2048, 1000)),
                                         (torch.bfloat16, (2100, 1000)), (torch.float32, (2300, 300)), (torch.float16, (2200, 999)),
                                         (torch.float64, (2050, 250)), (torch.int16, (2111, 1001))])
def test_reductions_many_short_rows_staged_in_shared_memory(dtype, shape):
    """Enough short rows to take the staged kernel (whole rows brought in by bulk copies, one
    thread per row); row counts that are not a multiple of the chunk exercise the ragged tail."""
    x = gen(shape, dtype, 60, -2.0, 2.0)
    dx = dev(x)
    for kind in ("argmax", "argmin", "max"):
        assert_same(getattr(tb, kind)(dx, -1), oracle.reduce(kind, x, -1))
    want_sum = oracle.reduce("sum", x, -1, acc=oracle.ACC_WIDE)
    if dtype in INTS:
        assert_same(tb.sum(dx, -1), want_sum)
    else:
        assert_close(tb.sum(dx, -1), want_sum)
        assert_close(tb.mean(dx, -1), oracle.reduce("mean", x, -1, acc=oracle.ACC_WIDE))
    mx, sm, am = tb.reduce_stats(dx, -1)
    assert_same(am, oracle.reduce("argmax", x, -1))
    assert_same(mx, oracle.reduce("max", x, -1))
    assert tb.device_errors() == 0


@pytest.mark.parametrize("dtype", HALVES)
@pytest.mark.parametrize("length", [197, 64, 33, 256, 510])
def test_staged_rows_ties_zeros_nan_and_infinities(dtype, length):
    """Short 16-bit rows are scanned two elements per instruction; only the group of the last strict
    improvement is remembered. Rows drawn from a handful of values put ties in every group; signed
    zeros, NaN and infinities are sprinkled in, and some rows hold nothing but -inf / NaN."""
    rows = 4200
    g = torch.Generator().manual_seed(length)
    palette = torch.tensor([-2.0, -1.0, -0.0, 0.0, 0.5, 1.0, 1.0, 3.0], dtype=torch.float32)
    x = palette[torch.randint(0, len(palette), (rows, length), generator=g)]
    special = torch.rand((rows, length), generator=g)
    x[special < 0.02] = float("nan")
    x[(special >= 0.02) & (special < 0.04)] = float("inf")
    x[(special >= 0.04) & (special < 0.06)] = float("-inf")
    x[7] = float("-inf")
    x[8] = float("nan")
    x[9] = float("-inf")
    x[9, length - 1] = float("nan")
    x[10, :] = -0.0
    x[10, length // 2] = 0.0        # +0 after -0: not greater, the first zero stays
    x[11, :] = -5.0
    x[11, length - 1] = -4.0        # the improvement sits in the very last element
    x[12, :] = -5.0
    x[12, 0] = -4.0                 # ... and in the very first
    x = x.to(dtype)
    dx = dev(x)
    for kind in ("argmax", "argmin"):
        assert_same(getattr(tb, kind)(dx, -1), oracle.reduce(kind, x, -1))
    got, want = tb.max(dx, -1).cpu(), oracle.reduce("max", x, -1)
    both_nan = torch.isnan(got.float()) & torch.isnan(want.float())
    assert torch.equal(got.view(torch.int16)[~both_nan], want.view(torch.int16)[~both_nan])
    mx, sm, am = tb.reduce_stats(dx, -1)
    assert_same(am, oracle.reduce("argmax", x, -1))
    # views that start on an odd element: every row is peeled by one
    v, dv = x[:, 1:], dx[:, 1:]
    assert_same(tb.argmax(dv.contiguous(), -1), oracle.reduce("argmax", v.contiguous(), -1))


def test_reduce_split_path_for_few_long_rows():
    x = gen((2, 1 << 20), torch.float32, 25, -1.0, 1.0)
    assert_close(tb.sum(dev(x), -1), oracle.reduce("sum", x, -1, acc=oracle.ACC_WIDE))
    assert_same(tb.argmax(dev(x), -1), oracle.reduce("argmax", x, -1))
    assert_close(tb.mean(dev(x), -1), oracle.reduce("mean", x, -1, acc=oracle.ACC_WIDE))


# ---------------------------------------------------------------- matmul ---------------

@pytest.mark.parametrize("pair", [(torch.float32, torch.float32), (torch.float64, torch.float64), (torch.int8, torch.int8),
                                  (torch.int32, torch.int32), (torch.int16, torch.int64), (torch.int32, torch.float32),
                                  (torch.bfloat16, torch.float32), (torch.float16, torch.float64)])
def test_matmul_simt_pairs(pair):
    a, b = gen((3, 37, 50), pair[0], 26, -1, 1), gen((3, 50, 29), pair[1], 27, -1, 1)
    want = oracle.matmul(a, b, acc=oracle.ACC_WIDE)
    got = tb.matmul(dev(a), dev(b))
    if want.dtype in INTS:
        assert_same(got, want)
    else:
        assert_close(got, want)


def test_matmul_config1_float32():
    """benchmark configuration 1: float32 [512,1024] x [1024,512], uniform[-1,1], seed 0."""
    a, b = oracle.fill((512, 1024), torch.float32, 0, "uniform", -1, 1), oracle.fill((1024, 512), torch.float32, 1000, "uniform", -1, 1)
    want = a.double() @ b.double()
    got = tb.matmul(dev(a), dev(b)).cpu()
    # summation order differs from the reference loop: arbitrate with the float64 product
    assert torch.allclose(got.double(), want, rtol=1e-4, atol=1e-4)
    sub = oracle.matmul(a[:16], b, acc=oracle.ACC_STORAGE)
    assert torch.allclose(got[:16], sub, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("dtype", HALVES)
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (128, 256, 256), (200, 300, 136), (197, 197, 64), (1, 8, 8), (130, 72, 1000), (384, 512, 4096)])
def test_matmul_tensor_core_k_major_b(dtype, m, n, k):
    """matmul(X, W.transpose(-1,-2)) with W [N, K]: both operands K-major."""
    a, w = gen((m, k), dtype, 28, -1, 1), gen((n, k), dtype, 29, -1, 1)
    want = oracle.matmul(a, w.t(), acc=oracle.ACC_WIDE)
    got = tb.matmul(dev(a), dev(w).t())
    assert_close(got, want)
    assert tb.device_errors() == 0


@pytest.mark.parametrize("dtype", HALVES)
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (100, 264, 200), (64, 3136, 256), (130, 8, 72)])
def test_matmul_tensor_core_n_major_b(dtype, m, n, k):
    """plain matmul(A, B) with B [K, N] row-major."""
    a, b = gen((m, k), dtype, 30, -1, 1), gen((k, n), dtype, 31, -1, 1)
    assert_close(tb.matmul(dev(a), dev(b)), oracle.matmul(a, b, acc=oracle.ACC_WIDE))
    assert tb.device_errors() == 0


def test_matmul_batched_broadcast_and_more_than_256_batches():
    """ViT-shaped scores: Q, K [b, 12, 197, 64]; more than 256 batches (the reference wraps there)."""
    q, k = gen((24, 12, 197, 64), torch.bfloat16, 32, -1, 1), gen((24, 12, 197, 64), torch.bfloat16, 33, -1, 1)
    got = tb.matmul(dev(q), dev(k).transpose(-1, -2), scale_by=0.125)
    assert got.shape == (24, 12, 197, 197)
    for i in (0, 11, 23):
        s = oracle.matmul(q[i], k[i].transpose(-1, -2), acc=oracle.ACC_WIDE)
        assert_close(got[i], oracle.scale(s, 0.125))
    # rank-4 x rank-2 broadcast (tests/cpu/test-matmul.cpp: Rank4Rank2StridedTransposed)
    x, w = gen((2, 3, 40, 64), torch.float16, 34, -1, 1), gen((48, 64), torch.float16, 35, -1, 1)
    assert_close(tb.matmul(dev(x), dev(w).t()), oracle.matmul(x, w.t(), acc=oracle.ACC_WIDE))
    # batch-broadcast first operand: one A for every batch of B
    a, b = gen((1, 40, 64), torch.float16, 36, -1, 1), gen((5, 64, 24), torch.float16, 37, -1, 1)
    assert_close(tb.matmul(dev(a), dev(b)), oracle.matmul(a, b, acc=oracle.ACC_WIDE))
    assert tb.device_errors() == 0


@pytest.mark.parametrize("dtype", HALVES)
def test_matmul_operand_broadcast_over_some_batch_dims(dtype):
    """[2,1,M,K] x [2,3,K,N]: the first operand's batch dims do not collapse into one stride over the six
    batches. The outermost batch dim is peeled off: one tensor-core launch per index, each over three batches."""
    a, b = gen((2, 1, 72, 64), dtype, 38, -1, 1), gen((2, 3, 64, 48), dtype, 39, -1, 1)
    launches = tb.launch_count()
    got = tb.matmul(dev(a), dev(b))
    assert tb.launch_count() - launches == 2
    assert got.shape == (2, 3, 72, 48)
    for i in range(2):
        for j in range(3):
            assert_close(got[i, j], oracle.matmul(a[i, 0], b[i, j], acc=oracle.ACC_WIDE))
    # the second operand broadcast instead, transposed (K-major) layout
    x, w = gen((3, 2, 40, 64), dtype, 40, -1, 1), gen((3, 1, 56, 64), dtype, 41, -1, 1)
    launches = tb.launch_count()
    got = tb.matmul(dev(x), dev(w).transpose(-1, -2))
    assert tb.launch_count() - launches == 3
    for i in range(3):
        for j in range(2):
            assert_close(got[i, j], oracle.matmul(x[i, j], w[i, 0].t(), acc=oracle.ACC_WIDE))
    assert tb.device_errors() == 0


@pytest.mark.parametrize("dtype", HALVES)
@pytest.mark.parametrize("batches,m,n,k,offset", [(5, 197, 197, 64, 0), (3, 300, 250, 128, 1), (7, 33, 7, 64, 3), (2, 128, 255, 192, 5),
                                                  (1, 5, 1, 8, 2), (9, 1, 33, 64, 7), (2, 260, 100, 320, 4)])
def test_matmul_rows_that_are_not_16_byte_multiples(dtype, batches, m, n, k, offset):
    """Dense results whose rows are an odd number of bytes from a 16-byte multiple leave the tensor-core
    kernel as one contiguous range per 32 rows (bulk store of the aligned middle, scalar head and tail).
    The result is placed `offset` elements into a larger buffer, so every alignment of its first byte
    is exercised, and the elements around it must stay untouched."""
    a, w = gen((batches, m, k), dtype, 62, -1, 1), gen((batches, n, k), dtype, 63, -1, 1)
    guard = 64
    flat = torch.full((guard + offset + batches * m * n + guard,), 7.0, dtype=dtype, device="cuda")
    out = flat[guard + offset:guard + offset + batches * m * n].view(batches, m, n)
    tb.matmul(dev(a), dev(w).transpose(-1, -2), scale_by=0.5, out=out)
    for i in sorted({0, batches - 1}):
        want = oracle.scale(oracle.matmul(a[i], w[i].t(), acc=oracle.ACC_WIDE), 0.5)
        assert_close(out[i], want)
    ref = torch.matmul(dev(a).float(), dev(w).float().transpose(-1, -2)) * 0.5
    assert torch.allclose(out.float(), ref, rtol=2e-2, atol=2e-2)
    assert bool((flat[:guard + offset] == 7.0).all()) and bool((flat[guard + offset + batches * m * n:] == 7.0).all())
    assert tb.device_errors() == 0


@pytest.mark.parametrize("n_major", [False, True])
@pytest.mark.parametrize("batches,m,n,k", [(1, 1024, 3136, 256), (3, 300, 520, 192), (400, 197, 197, 64), (2, 2000, 264, 128), (170, 256, 256, 256)])
def test_matmul_short_k_many_row_tiles(batches, m, n, k, n_major):
    """K of at most 256 with several row tiles and many tiles per CTA: short main loops, so the
    epilogue and the accumulator hand-over set the pace; ragged edges in both directions."""
    dtype = torch.bfloat16 if n_major else torch.float16
    a = gen((batches, m, k), dtype, 60, -1, 1)
    if n_major:
        b = gen((batches, k, n), dtype, 61, -1, 1)
        got = tb.matmul(dev(a), dev(b))
        pick = lambda i, r: oracle.matmul(a[i][r], b[i], acc=oracle.ACC_WIDE)
    else:
        w = gen((batches, n, k), dtype, 61, -1, 1)
        got = tb.matmul(dev(a), dev(w).transpose(-1, -2))
        pick = lambda i, r: oracle.matmul(a[i][r], w[i].t(), acc=oracle.ACC_WIDE)
    rows = slice(0, m) if m * n * k <= 300 * 520 * 192 else slice(m - 160, m)
    for i in sorted({0, batches // 2, batches - 1}):
        assert_close(got[i][rows], pick(i, rows))
    # every batch against a float32 product on the device (loose: catches a misplaced tile)
    ref = torch.matmul(dev(a).float(), dev(b).float() if n_major else dev(w).float().transpose(-1, -2))
    assert torch.allclose(got.float(), ref, rtol=2e-2, atol=2e-2)
    assert tb.device_errors() == 0


@pytest.mark.parametrize("dtype,m,k,n,batches,lda,scale", [
    (torch.float16, 200, 256, 824, 600, None, None),    # two row tiles (the second ragged), last column tile 56 wide
    (torch.bfloat16, 128, 64, 1000, 1000, None, 0.5),   # one K block, one row tile: 148 groups
    (torch.float16, 200, 75, 816, 600, 80, None),       # K not a multiple of 8 inside a wider pitch: the tail of A must read as zero
    (torch.float16, 1024, 256, 3136, 48, None, None),   # the 1x1-convolution geometry: eight row tiles, 18 groups
    (torch.bfloat16, 300, 136, 200, 1000, None, None),  # three row tiles, two column tiles per batch
])
def test_matmul_short_k_shared_first_operand(dtype, m, k, n, batches, lda, scale):
    """One A[M, K <= 256] against many B[K, N] (N contiguous) with enough column tiles: the kernel
    that keeps A in tensor memory and streams only B. Selected batches against the oracle, all of
    them against a float32 product on the device."""
    a_full = gen((m, lda or k), dtype, 70, -1, 1)
    a = a_full[:, :k]
    b = gen((batches, k, n), dtype, 71, -1, 1)
    da = dev(a_full)[:, :k]
    before = tb.gemm_path_launches()["stationary"]
    got = tb.matmul(da, dev(b)) if scale is None else tb.matmul(da, dev(b), scale_by=scale)
    assert tb.gemm_path_launches()["stationary"] == before + 1, "this shape is meant for the stationary-A kernel"
    assert got.shape == (batches, m, n)
    rows = slice(m - 72, m)
    for i in sorted({0, batches // 2, batches - 1}):
        want = oracle.matmul(a[rows].contiguous(), b[i], acc=oracle.ACC_WIDE)
        assert_close(got[i][rows], want if scale is None else oracle.scale(want, scale))
    for lo in range(0, batches, 100):  # every batch against a float32 product on the device, a slab at a time
        ref = torch.matmul(da.float(), dev(b[lo:lo + 100]).float()) * (scale or 1.0)
        assert torch.allclose(got[lo:lo + 100].float(), ref, rtol=2e-2, atol=2e-2 * (4 if dtype == torch.bfloat16 else 1))
    assert tb.device_errors() == 0


@pytest.mark.parametrize("dtype", HALVES)
@pytest.mark.parametrize("shape", [
    # (N, Cin, H, W, Cout, Kh, Kw, stride, pad)
    (2, 3, 64, 64, 16, 7, 7, 2, 3),      # a ResNet-stem geometry: three input channels
    (3, 20, 18, 24, 40, 3, 3, 1, 1),     # 20 channels: padded to 24
    (1, 67, 12, 16, 8, 3, 3, 1, 0),      # two channel blocks, the second holds 3 real + 5 zero channels
])
def test_conv2d_channel_counts_that_are_not_multiples_of_8(dtype, shape):
    """The NHWC copy and the packed weights pad the channel pitch to a multiple of 8 with zeros, so these
    convolutions run on the tensor cores too (they used to fall to the one-thread-per-output kernel)."""
    n, cin, h, w, cout, kh, kw, stride, pad = shape
    x = gen((n, cin, h, w), dtype, 55, -1, 1)
    wt = gen((cout, cin, kh, kw), dtype, 56, -0.2, 0.2)
    bias = gen((cout,), dtype, 57, -1, 1)
    before = tb.gemm_path_launches()["general"]
    got = tb.convolve2D(dev(x), dev(wt), stride, pad, bias=dev(bias))
    assert tb.gemm_path_launches()["general"] == before + 1, "expected the implicit GEMM"
    assert_close(got, oracle.conv2d(x, wt, stride, pad, bias=bias, acc=oracle.ACC_WIDE))
    assert tb.device_errors() == 0


@pytest.mark.parametrize("dtype", HALVES)
@pytest.mark.parametrize("shape", [(2, 64, 20, 24, 40, 3, 3, 1, 1), (2, 3, 32, 32, 16, 5, 5, 2, 2), (3, 72, 9, 16, 8, 1, 1, 1, 0)])
def test_conv2d_with_weights_packed_ahead(dtype, shape):
    """tn_conv2d_pack_weights + tn_conv2d_prepacked give the bits of tn_conv2d (with and without bias), the packed
    copy is reusable, and the call that uses it launches no weight packing of its own."""
    n, cin, h, w, cout, kh, kw, stride, pad = shape
    x = dev(gen((n, cin, h, w), dtype, 58, -1, 1))
    wt = dev(gen((cout, cin, kh, kw), dtype, 59, -0.2, 0.2))
    bias = dev(gen((cout,), dtype, 60, -1, 1))
    packed = tb.pack_conv_weights(wt)
    assert packed is not None and packed.numel() == kh * kw * cout * ((cin + 7) // 8 * 8)
    for b in (None, bias):
        want = tb.convolve2D(x, wt, stride, pad, bias=b)
        for _ in range(2):
            got = tb.convolve2D(x, wt, stride, pad, bias=b, packed=packed)
            assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    assert tb.pack_conv_weights(dev(gen((4, 3, 3, 3), torch.float32, 61, -1, 1))) is None
    assert tb.device_errors() == 0


@pytest.mark.parametrize("dtype", HALVES)
def test_conv2d_1x1_many_images_with_bias(dtype):
    """1x1 convolution on NCHW with enough images for the stationary-weights kernel; bias per output channel."""
    x = gen((336, 72, 40, 40), dtype, 72, -1, 1)
    wt = gen((200, 72, 1, 1), dtype, 73, -0.2, 0.2)
    bias = gen((200,), dtype, 74, -1, 1)
    before = tb.gemm_path_launches()["stationary"]
    got = tb.convolve2D(dev(x), dev(wt), 1, 0, bias=dev(bias))
    assert tb.gemm_path_launches()["stationary"] == before + 1
    for i in (0, 170, 335):
        assert_close(got[i:i + 1], oracle.conv2d(x[i:i + 1], wt, 1, 0, bias=bias, acc=oracle.ACC_WIDE))
    ref = torch.nn.functional.conv2d(dev(x).float(), dev(wt).float(), dev(bias).float())
    assert torch.allclose(got.float(), ref, rtol=2e-2, atol=3e-2)
    assert tb.device_errors() == 0


@pytest.mark.parametrize("case", ["plain", "b_transposed", "a_transposed", "batched", "shared_b", "odd"])
def test_matmul_float32_on_tensor_cores(case):
    """float32 products above 2^24 multiply-adds run on the tensor cores: each operand is split into three
    bfloat16 parts and the six significant part products are summed in float32. Checked against the float64
    product (summation order differs from the reference loop) and, on a block of rows, against the oracle."""
    if case == "plain":
        a, b = gen((384, 520), torch.float32, 90, -1, 1), gen((520, 300), torch.float32, 91, -1, 1)
        da, db = dev(a), dev(b)
    elif case == "b_transposed":
        a, w = gen((256, 1024), torch.float32, 92, -1, 1), gen((136, 1024), torch.float32, 93, -1, 1)
        b = w.t()
        da, db = dev(a), dev(w).t()
    elif case == "a_transposed":
        at, b = gen((512, 200), torch.float32, 94, -1, 1), gen((512, 264), torch.float32, 95, -1, 1)
        a = at.t()
        da, db = dev(at).t(), dev(b)
    elif case == "batched":
        a, b = gen((5, 130, 333), torch.float32, 96, -1, 1), gen((5, 333, 200), torch.float32, 97, -1, 1)
        da, db = dev(a), dev(b)
    elif case == "shared_b":
        a, b = gen((3, 4, 100, 256), torch.float32, 98, -1, 1), gen((256, 192), torch.float32, 99, -1, 1)
        da, db = dev(a), dev(b)
    else:
        a, b = gen((257, 1001), torch.float32, 100, -50, 50), gen((1001, 67), torch.float32, 101, -1e-3, 1e-3)
        da, db = dev(a), dev(b)
    launches = tb.launch_count()
    got = tb.matmul(da, db)
    assert tb.launch_count() - launches == 4, "expected two split passes, the tensor-core GEMM and the (idle) fallback"
    want = torch.matmul(a.double(), b.double())
    scale = torch.matmul(a.double().abs(), b.double().abs())  # size of the terms that were summed
    assert got.dtype == torch.float32 and got.shape == want.shape
    assert bool(((got.cpu().double() - want).abs() <= 4e-6 * scale + 1e-30).all())
    rows = oracle.matmul(a.reshape(-1, a.shape[-2], a.shape[-1])[0][:8], b.reshape(-1, b.shape[-2], b.shape[-1])[0], acc=oracle.ACC_STORAGE)
    assert torch.allclose(got.reshape(-1, got.shape[-2], got.shape[-1])[0][:8].cpu(), rows, rtol=1e-4, atol=1e-4 * float(scale.max()))
    assert tb.device_errors() == 0
    # infinities and NaN cannot be split: the passes flag them and the element-wise kernel recomputes on the device
    a2 = a.clone().reshape(-1, a.shape[-1])
    a2[0, 0], a2[1, 1] = float("inf"), 3.0e38
    a2 = a2.reshape(a.shape)
    out = tb.matmul(dev(a2) if case != "a_transposed" else dev(a2.t().contiguous()).t(), db).cpu()
    ref = torch.matmul(a2.double(), b.double()).float()
    assert torch.isinf(out.reshape(-1, out.shape[-1])[0]).all() and torch.equal(torch.isinf(out), torch.isinf(ref))


@pytest.mark.parametrize("dtype", HALVES)
@pytest.mark.parametrize("case", ["a_transposed", "both_transposed", "b_strided", "odd_pitch", "batched_a_transposed"])
def test_matmul_half_operands_in_any_layout_reach_the_tensor_cores(dtype, case):
    """tests/cpu/test-matmul.cpp BothTransposed and friends, at sizes where it matters: operands the TMA
    maps cannot address are copied dense first (tiled transpose), then take the tcgen05 path."""
    if case == "a_transposed":
        at, b = gen((512, 264), dtype, 110, -1, 1), gen((512, 320), dtype, 111, -1, 1)
        a, da, db = at.t(), dev(at).t(), dev(b)
    elif case == "both_transposed":
        at, bt = gen((256, 300), dtype, 112, -1, 1), gen((264, 256), dtype, 113, -1, 1)
        a, b, da, db = at.t(), bt.t(), dev(at).t(), dev(bt).t()
    elif case == "b_strided":
        a, b0 = gen((300, 512), dtype, 114, -1, 1), gen((512, 528), dtype, 115, -1, 1)
        b, da, db = b0[:, ::2], dev(a), dev(b0)[:, ::2]
    elif case == "odd_pitch":
        a0, b = gen((300, 1001), dtype, 116, -1, 1), gen((512, 200), dtype, 117, -1, 1)
        a, da, db = a0[:, :512], dev(a0)[:, :512], dev(b)
    else:
        at, b = gen((6, 128, 200), dtype, 118, -1, 1), gen((6, 128, 136), dtype, 119, -1, 1)
        a, da, db = at.transpose(-1, -2), dev(at).transpose(-1, -2), dev(b)
    launches = tb.launch_count()
    got = tb.matmul(da, db)
    assert tb.launch_count() - launches >= 2, "expected a staging copy in front of the tensor-core GEMM"
    a3, b3, g3 = (t.reshape((-1,) + tuple(t.shape[-2:])) for t in (a, b, got.cpu()))
    for i in sorted({0, a3.shape[0] - 1}):
        # the reference loop reads an operand through max(stride) alone (src/cpu/matmul.cpp:126-176), so it is
        # given dense copies of views whose inner stride is not 1
        assert_close(g3[i][:24], oracle.matmul(a3[i][:24].contiguous(), b3[i].contiguous(), acc=oracle.ACC_WIDE))
    ref = torch.matmul(da.float(), db.float())
    assert torch.allclose(got.float(), ref, rtol=2e-2, atol=2e-2)
    assert tb.device_errors() == 0


def test_matmul_half_to_float32_result():
    a, w = gen((130, 136), torch.bfloat16, 38, -1, 1), gen((72, 136), torch.bfloat16, 39, -1, 1)
    got = tb.matmul(dev(a), dev(w).t(), out_dtype=A.FLOAT32)
    want = oracle.matmul(a, w.t(), acc=oracle.ACC_WIDE, out_dtype=A.FLOAT32)
    assert_close(got, want, tol=(1e-4, 1e-4))


def test_matmul_short_k_shared_first_operand_float32_result():
    """The kernel that keeps A in tensor memory, writing float32 (16 elements per store box instead of 32)."""
    a, b = gen((136, 128), torch.bfloat16, 75, -1, 1), gen((500, 128, 1000), torch.bfloat16, 76, -1, 1)
    before = tb.gemm_path_launches()["stationary"]
    got = tb.matmul(dev(a), dev(b), out_dtype=A.FLOAT32)
    assert tb.gemm_path_launches()["stationary"] == before + 1
    assert got.dtype == torch.float32 and got.shape == (500, 136, 1000)
    for i in (0, 131, 499):
        assert_close(got[i], oracle.matmul(a, b[i], acc=oracle.ACC_WIDE, out_dtype=A.FLOAT32), tol=(1e-4, 1e-4))
    ref = torch.matmul(dev(a).float(), dev(b).float())
    assert torch.allclose(got, ref, rtol=1e-3, atol=1e-3)
    assert tb.device_errors() == 0


def test_matmul_with_an_sm_margin():
    """tn_set_sm_margin: the persistent tensor-core kernels run on fewer SMs and give the same bits."""
    a, w = gen((3, 700, 256), torch.bfloat16, 77, -1, 1), gen((3, 520, 256), torch.bfloat16, 78, -1, 1)
    x = gen((4, 64, 30, 40), torch.float16, 79, -1, 1)
    k = gen((48, 64, 3, 3), torch.float16, 80, -0.2, 0.2)
    want = tb.matmul(dev(a), dev(w).transpose(-1, -2))
    want_conv = tb.convolve2D(dev(x), dev(k), 1, 1)
    try:
        for margin in (1, 32, 64):
            tb.sm_margin(margin)
            assert torch.equal(tb.matmul(dev(a), dev(w).transpose(-1, -2)).view(torch.int16), want.view(torch.int16))
            assert torch.equal(tb.convolve2D(dev(x), dev(k), 1, 1).view(torch.int16), want_conv.view(torch.int16))
        with pytest.raises(A.TannicError):
            tb.sm_margin(65)
        with pytest.raises(A.TannicError):
            tb.sm_margin(-1)
    finally:
        tb.sm_margin(0)
    assert_close(want[1], oracle.matmul(a[1], w[1].t(), acc=oracle.ACC_WIDE))
    assert tb.device_errors() == 0


def test_matmul_errors():
    a, b = dev(gen((4, 5), torch.float16, 1)), dev(gen((5, 3), torch.bfloat16, 2))
    with pytest.raises(A.TannicError) as e:
        tb.matmul(a, b, out_dtype=A.FLOAT16)
    assert e.value.status == A.UNSUPPORTED_DTYPE


# ---------------------------------------------------------------- data movement --------

@pytest.mark.parametrize("pair", [(torch.float32, torch.float32), (torch.float16, torch.float16), (torch.bfloat16, torch.float32),
                                  (torch.int32, torch.int32), (torch.int8, torch.int64), (torch.float64, torch.int32)])
def test_outer(pair):
    a, b = gen((37,), pair[0], 70, -2, 2), gen((53,), pair[1], 71, -2, 2)
    want = oracle.outer(a, b)
    got = tb.outer(dev(a), dev(b))
    (assert_same if want.dtype in INTS or pair[0] == pair[1] else assert_close)(got, want)
    assert_same(tb.outer(dev(a)[::2], dev(b)[1::3]), oracle.outer(a[::2], b[1::3])) if pair[0] == pair[1] else None


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int8, torch.int64, torch.float64])
@pytest.mark.parametrize("axis", [0, 1, 2, -1])
def test_repeat(dtype, axis):
    x = gen((5, 6, 7), dtype, 72)
    assert_same(tb.repeat(dev(x), 3, axis), oracle.repeat(x, 3, axis))
    assert_same(tb.repeat(dev(x).transpose(0, 2), 2, axis), oracle.repeat(x.transpose(0, 2), 2, axis))  # tests/cpu/test-repeats.cpp: after permute
    assert_same(tb.repeat(dev(x), 1, axis), x)
    big = gen((64, 129, 33), dtype, 73)
    assert_same(tb.repeat(dev(big), 4, 1), torch.repeat_interleave(big, 4, 1))
    wide = gen((16, 24, 64), dtype, 74)  # inner runs that move as 16-byte words
    assert_same(tb.repeat(dev(wide), 3, 1), torch.repeat_interleave(wide, 3, 1))
    assert_same(tb.repeat(dev(wide), 2, 0), torch.repeat_interleave(wide, 2, 0))


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.int32, torch.float64])
def test_concat(dtype):
    a, b = gen((3, 4, 5), dtype, 74), gen((2, 4, 5), dtype, 75)
    assert_same(tb.concatenate(dev(a), dev(b), 0), oracle.concat(a, b, 0))  # the axis the reference's CPU loop gets wrong
    c = gen((3, 9, 5), dtype, 76)
    assert_same(tb.concatenate(dev(a), dev(c), 1), oracle.concat(a, c, 1))
    d = gen((3, 4, 1), dtype, 77)
    assert_same(tb.concatenate(dev(a), dev(d), -1), oracle.concat(a, d, 2))
    m, n = gen((40, 64), dtype, 78), gen((24, 64), dtype, 79)
    assert_same(tb.concatenate(dev(m).t(), dev(n).t(), 1), oracle.concat(m.t(), n.t(), 1))
    big_a, big_b = gen((300, 1000), dtype, 80), gen((300, 24), dtype, 81)
    assert_same(tb.concatenate(dev(big_a), dev(big_b), 1), torch.cat([big_a, big_b], 1))
    with pytest.raises(ValueError):
        tb.concatenate(dev(a), dev(b).to(torch.int16), 0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16, torch.int32, torch.int64, torch.float64, torch.int8])
@pytest.mark.parametrize("k", [-3, -1, 0, 1, 4])
def test_triangular_masks(dtype, k):
    m = gen((33, 47), dtype, 82)
    assert_same(tb.triu(dev(m), k), oracle.triangular(m, True, k))
    assert_same(tb.tril(dev(m), k), oracle.triangular(m, False, k))
    assert_same(tb.triu(dev(m).t(), k), oracle.triangular(m.t(), True, k))
    assert_same(tb.tril(dev(m), k), torch.tril(m, k))
    with pytest.raises(A.TannicError):
        tb.triu(dev(gen((2, 3, 4), dtype, 83)), k)


@pytest.mark.parametrize("pair", [(torch.float32, torch.float32), (torch.float64, torch.float64), (torch.float32, torch.float64)])
def test_complex_constructors(pair):
    rho, theta = gen((6, 1, 33), pair[0], 84, 0, 2), gen((1, 7, 33), pair[1], 85, -3, 3)
    got = tb.cartesian(dev(rho), dev(theta)).cpu()
    assert torch.equal(torch.view_as_real(got), torch.view_as_real(oracle.complex_pair(rho, theta, False)))
    got = tb.polar(dev(rho), dev(theta)).cpu()
    want = oracle.complex_pair(rho, theta, True)
    tol = 1e-12 if torch.float64 in pair else 1e-5
    assert torch.allclose(torch.view_as_real(got), torch.view_as_real(want), rtol=tol, atol=tol)
    # tests/cuda/test-cuda-complex.cpp: integer radii are accepted by polar
    r = oracle.fill((4, 5), torch.int32, 86, "uniform", -5, 5)
    t = gen((4, 5), torch.float32, 87, -3, 3)
    assert torch.allclose(torch.view_as_real(tb.polar(dev(r), dev(t)).cpu()), torch.view_as_real(torch.polar(r.float(), t)), rtol=1e-5, atol=1e-5)
    # complex arithmetic on the results (same-type complex add / mul)
    z = tb.polar(dev(rho), dev(theta))
    assert torch.allclose(torch.view_as_real(tb.mul(z, z).cpu()), torch.view_as_real(want * want), rtol=1e-4 if torch.float64 not in pair else 1e-10, atol=1e-5)


# ---------------------------------------------------------------- conv2d ---------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16, torch.float64, torch.int32])
@pytest.mark.parametrize("stride,padding", [(1, 0), (1, 1), (2, 1), ((2, 1), (0, 2))])
def test_conv2d_direct(dtype, stride, padding):
    x, w = gen((2, 5, 9, 8), dtype, 40, -1, 1), gen((6, 5, 3, 2), dtype, 41, -1, 1)
    bias = gen((6,), dtype, 42, -1, 1)
    want = oracle.conv2d(x, w, stride, padding, acc=oracle.ACC_WIDE)
    got = tb.convolve2D(dev(x), dev(w), stride, padding)
    if dtype in INTS:
        assert_same(got, want)
    else:
        assert_close(got, want)
    wantb = oracle.conv2d(x, w, stride, padding, bias=bias, acc=oracle.ACC_WIDE)
    gotb = tb.convolve2D(dev(x), dev(w), stride, padding, bias=dev(bias))
    assert_same(gotb, wantb) if dtype in INTS else assert_close(gotb, wantb)


@pytest.mark.parametrize("dtype", HALVES)
def test_conv2d_1x1_tensor_core(dtype):
    x, w = gen((3, 64, 12, 12), dtype, 43, -1, 1), gen((40, 64, 1, 1), dtype, 44, -1, 1)
    bias = gen((40,), dtype, 45, -1, 1)
    assert_close(tb.convolve2D(dev(x), dev(w), 1, 0), oracle.conv2d(x, w, 1, 0, acc=oracle.ACC_WIDE))
    assert_close(tb.convolve2D(dev(x), dev(w), 1, 0, bias=dev(bias)), oracle.conv2d(x, w, 1, 0, bias=bias, acc=oracle.ACC_WIDE))
    assert tb.device_errors() == 0


@pytest.mark.parametrize("dtype", HALVES)
@pytest.mark.parametrize("shape", [
    # (N, Cin, H, W, Cout, Kh, Kw, pad)
    (2, 64, 14, 14, 32, 3, 3, 1),       # one pixel tile per image, one channel block
    (3, 72, 20, 24, 136, 3, 3, 1),      # ragged channel block (72 = 64 + 8), two Cout tiles, ragged last row tile
    (1, 128, 56, 56, 64, 3, 3, 1),      # ResNet-stage geometry: 4 output rows (224 pixels) per tile
    (2, 16, 9, 40, 8, 3, 5, 0),         # no padding, rectangular kernel
    (2, 32, 12, 12, 16, 5, 5, 2),       # 25 taps
    (1, 8, 70, 250, 24, 3, 3, 2),       # one output row per tile (Wout = 252), padding 2
])
def test_conv2d_implicit_gemm_tensor_core(dtype, shape):
    n, cin, h, w, cout, kh, kw, pad = shape
    x = gen((n, cin, h, w), dtype, 47, -1, 1)
    wt = gen((cout, cin, kh, kw), dtype, 48, -0.2, 0.2)
    bias = gen((cout,), dtype, 49, -1, 1)
    want = oracle.conv2d(x, wt, 1, pad, acc=oracle.ACC_WIDE)
    assert_close(tb.convolve2D(dev(x), dev(wt), 1, pad), want)
    assert_close(tb.convolve2D(dev(x), dev(wt), 1, pad, bias=dev(bias)), oracle.conv2d(x, wt, 1, pad, bias=bias, acc=oracle.ACC_WIDE))
    assert tb.device_errors() == 0


@pytest.mark.parametrize("dtype", HALVES)
@pytest.mark.parametrize("shape", [
    # (N, Cin, H, W, Cout, Kh, Kw, stride, pad)
    (2, 64, 56, 56, 128, 3, 3, 2, 1),        # ResNet stage entry: 3x3 stride 2
    (2, 256, 28, 28, 136, 1, 1, 2, 0),       # ResNet downsample: 1x1 stride 2
    (1, 16, 33, 47, 24, 3, 3, (2, 3), 1),    # different strides per axis, odd extents
    (2, 8, 30, 30, 16, 7, 7, 2, 3),          # 49 taps, stride 2, padding 3
    (1, 32, 40, 40, 8, 3, 3, 4, 0),          # stride 4
])
def test_conv2d_strided_on_tensor_cores(dtype, shape):
    """Stride > 1 through the implicit GEMM: the activation's tensor map walks W and H with the
    convolution's stride, every other part of the kernel is the stride-1 one."""
    n, cin, h, w, cout, kh, kw, stride, pad = shape
    x = gen((n, cin, h, w), dtype, 52, -1, 1)
    wt = gen((cout, cin, kh, kw), dtype, 53, -0.2, 0.2)
    bias = gen((cout,), dtype, 54, -1, 1)
    launches = tb.launch_count()
    got = tb.convolve2D(dev(x), dev(wt), stride, pad)
    # staging (the weight re-layout rides along in the same launch when the activation is dense) + tensor-core GEMM
    assert tb.launch_count() - launches in (2, 3), "expected staging (+ weight packing) + tensor-core GEMM"
    assert_close(got, oracle.conv2d(x, wt, stride, pad, acc=oracle.ACC_WIDE))
    assert_close(tb.convolve2D(dev(x), dev(wt), stride, pad, bias=dev(bias)), oracle.conv2d(x, wt, stride, pad, bias=bias, acc=oracle.ACC_WIDE))
    assert tb.device_errors() == 0


def test_conv2d_implicit_gemm_strided_input_view():
    x = gen((2, 12, 10, 64), torch.float16, 50, -1, 1)            # [N, H, W, C] storage
    xv = x.permute(0, 3, 1, 2)                                     # NCHW view with channel stride 1
    wt = gen((16, 64, 3, 3), torch.float16, 51, -0.2, 0.2)
    want = oracle.conv2d(xv, wt, 1, 1, acc=oracle.ACC_WIDE)
    launches = tb.launch_count()
    got = tb.convolve2D(dev(x).permute(0, 3, 1, 2), dev(wt), 1, 1)
    assert tb.launch_count() - launches == 2, "channels-last storage is read in place: weight packing + GEMM only"
    assert_close(got, want)
    # a view that is neither NCHW-dense nor channels-last goes through the generic staging kernel
    xs = gen((2, 64, 12, 20), torch.float16, 55, -1, 1)
    assert_close(tb.convolve2D(dev(xs)[:, :, :, ::2], dev(wt), 1, 1), oracle.conv2d(xs[:, :, :, ::2], wt, 1, 1, acc=oracle.ACC_WIDE))


def test_conv2d_errors():
    x, w = dev(gen((1, 3, 5, 5), torch.float32, 1)), dev(gen((2, 4, 3, 3), torch.float32, 2))
    y = torch.empty(1, 2, 3, 3, device="cuda")
    import ctypes as C
    dx, dw, dy = tb.desc(x), tb.desc(w), tb.desc(y)
    pad, strd = (C.c_size_t * 2)(0, 0), (C.c_size_t * 2)(1, 1)
    assert A.lib().tn_conv2d(C.byref(dx), C.byref(dw), C.byref(dy), tb.current_stream(x), pad, strd) == A.ERROR
    w16 = dev(gen((2, 3, 3, 3), torch.float16, 2))
    dw16 = tb.desc(w16)
    assert A.lib().tn_conv2d(C.byref(dx), C.byref(dw16), C.byref(dy), tb.current_stream(x), pad, strd) == A.UNSUPPORTED_DTYPE


# ---------------------------------------------------------------- runtime / utilities ---

def test_cpy_and_allclose():
    x = gen((20, 30), torch.float32, 46)
    dst = torch.zeros(30, 20, device="cuda")
    tb.cpy(dev(x).t(), dst)
    assert torch.equal(dst.cpu(), x.t().contiguous())
    dx = dev(x)
    assert tb.allclose(dx, dx.clone())
    y = dx.clone()
    y[3, 4] += 1.0
    assert not tb.allclose(dx, y)
    assert tb.allclose(dx, y, rtol=0.0, atol=2.0)


def test_allocator_streams_and_copies():
    import ctypes as C
    lib = A.lib()
    n = C.c_int(0)
    A.check(lib.tn_device_count(C.byref(n)))
    assert n.value >= 1
    d = A.DeviceT(0)
    ptrs = []
    for _ in range(5):  # tests/cuda/test-cuda-allocations.cpp: five allocations, then frees
        p = C.c_void_p()
        A.check(lib.tn_allocate(C.byref(d), 1 << 20, C.byref(p)))
        assert p.value
        ptrs.append(p)
    host = torch.arange(1 << 18, dtype=torch.int32)
    A.check(lib.tn_copy_from_host(C.byref(d), host.data_ptr(), ptrs[0], host.numel() * 4))
    back = torch.zeros_like(host)
    A.check(lib.tn_copy_to_host(C.byref(d), ptrs[0], back.data_ptr(), host.numel() * 4))
    assert torch.equal(host, back)
    eq = C.c_int(0)
    A.check(lib.tn_compare_from_host(C.byref(d), host.data_ptr(), ptrs[0], host.numel() * 4, C.byref(eq)))
    assert eq.value == 1
    for p in ptrs:
        A.check(lib.tn_deallocate(C.byref(d), p))
    s1, s2 = A.StreamT(), A.StreamT()
    A.check(lib.tn_stream_pop(C.byref(d), C.byref(s1)))
    A.check(lib.tn_stream_put(C.byref(d), s1))
    A.check(lib.tn_stream_pop(C.byref(d), C.byref(s2)))
    assert s1.address == s2.address and s1.address != 0  # LIFO: the same stream comes back
    # stream-ordered copies through pinned host memory
    hp, hq, dp = C.c_void_p(), C.c_void_p(), C.c_void_p()
    nbytes = host.numel() * 4
    A.check(lib.tn_host_allocate_pinned(nbytes, C.byref(hp)))
    A.check(lib.tn_host_allocate_pinned(nbytes, C.byref(hq)))
    A.check(lib.tn_allocate(C.byref(d), nbytes, C.byref(dp)))
    C.memmove(hp, host.data_ptr(), nbytes)
    A.check(lib.tn_copy_from_host_async(C.byref(d), hp, dp, nbytes, s2))
    A.check(lib.tn_copy_to_host_async(C.byref(d), dp, hq, nbytes, s2))
    A.check(lib.tn_stream_synchronize(s2))
    got = torch.zeros_like(host)
    C.memmove(got.data_ptr(), hq, nbytes)
    assert torch.equal(got, host)
    A.check(lib.tn_deallocate(C.byref(d), dp))
    A.check(lib.tn_host_free_pinned(hp))
    A.check(lib.tn_host_free_pinned(hq))
    A.check(lib.tn_stream_put(C.byref(d), s2))
    bad = A.DeviceT(99)
    p = C.c_void_p()
    assert lib.tn_allocate(C.byref(bad), 16, C.byref(p)) == A.ERROR


def test_host_tensor_is_rejected_without_fallback():
    a = gen((4,), torch.float32, 1)
    with pytest.raises(A.TannicError) as e:
        _add_host(a)
    assert e.value.status == A.INCOMPATIBLE_DEVICES


def _add_host(a):
    import ctypes as C
    out = torch.empty_like(a)
    da, dd = tb.desc(a), tb.desc(out)
    A.check(A.lib().tn_add(C.byref(da), C.byref(da), C.byref(dd), A.StreamT(0)))



# ---------------------------------------------------------------- comparisons, conv1d ---

@pytest.mark.parametrize("dtype", INTS + FLOATS)
@pytest.mark.parametrize("op", list(oracle.COMPARE))
def test_comparisons_bit_packed(dtype, op):
    """eq / ne / gt / ge / lt / le on the device: the packed bytes equal the oracle's, dense and strided
    operands, ragged sizes (padding bits zero), NaN and infinities, and a broadcast operand."""
    for shape in ((1000,), (3, 5, 7), (64, 33)):
        a, b = gen(shape, dtype, 80), gen(shape, dtype, 81)
        b.view(-1)[::3] = a.view(-1)[::3]
        if dtype not in INTS:
            a.view(-1)[5] = float("nan")
            b.view(-1)[7] = float("inf")
            a.view(-1)[9] = float("-inf")
        want, _ = oracle.compare_packed(op, a, b)
        got = getattr(tb, op)(dev(a), dev(b))
        assert torch.equal(got.cpu(), want), (shape,)
    a, b = gen((6, 40), dtype, 82), gen((40, 6), dtype, 83)
    want, _ = oracle.compare_packed(op, a, b.t())
    assert torch.equal(getattr(tb, op)(dev(a), dev(b).t()).cpu(), want)
    row = gen((1, 40), dtype, 84)
    want, shape = oracle.compare_packed(op, a, row)
    got = getattr(tb, op)(dev(a), dev(row))
    assert torch.equal(got.cpu(), want)
    assert torch.equal(tb.unpack_bits(got, shape), oracle.compare(op, a, row))


def test_comparison_rejects_mixed_dtypes_and_non_boolean_results():
    a, b = dev(gen((4, 4), torch.float32, 85)), dev(gen((4, 4), torch.float16, 86))
    with pytest.raises(A.TannicError):
        tb.eq(a, b)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32, torch.float64, torch.int32])
@pytest.mark.parametrize("n,c,l,cout,k,stride,pad", [(2, 3, 19, 4, 5, 1, 0), (1, 8, 200, 16, 3, 2, 1), (3, 16, 64, 8, 7, 3, 3), (2, 64, 1000, 32, 3, 1, 1)])
def test_conv1d_generated_shapes(dtype, n, c, l, cout, k, stride, pad):
    """conv1d against the oracle (the reference's loop nest with float accumulation for 16-bit types);
    the last shape is large enough for the tensor-core path of the H = 1 convolution."""
    x, w = gen((n, c, l), dtype, 87, -1, 1), gen((cout, c, k), dtype, 88, -0.5, 0.5)
    want = oracle.conv1d(x, w, stride, pad, acc=oracle.ACC_WIDE)
    got = tb.convolve1D(dev(x), dev(w), stride, pad)
    if dtype in INTS:
        assert_same(got, want)
    else:
        assert_close(got, want)
    assert tb.device_errors() == 0


# ---------------------------------------------------------------- bulk initialisation ---

def test_element_assignments_leave_as_one_copy():
    """tn_assign_from_host: 1000 element-sized writes to consecutive addresses (what Tensor::assign does
    for an initializer list, src/tensor.cpp:34-44) become one host-to-device copy, issued when the thread
    enters another entry point; a gap starts a new run; the values arrive in order."""
    import ctypes as C
    lib = A.lib()
    dev0 = A.DeviceT(torch.cuda.current_device())
    target = torch.zeros(1000, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    values = torch.arange(1000, dtype=torch.float32) * 0.5
    before = lib.tn_h2d_copy_count()
    for i in range(1000):
        A.check(lib.tn_assign_from_host(C.byref(dev0), values.data_ptr() + 4 * i, target.data_ptr() + 4 * i, 4))
    assert lib.tn_h2d_copy_count() == before          # nothing has left yet
    host = torch.empty(1000, dtype=torch.float32)
    A.check(lib.tn_copy_to_host(C.byref(dev0), target.data_ptr(), host.data_ptr(), 4000))   # flushes, then reads back
    assert lib.tn_h2d_copy_count() == before + 1
    assert torch.equal(host, values)
    # two runs with a gap between them: two copies; an op on the tensor sees both
    target.zero_()
    torch.cuda.synchronize()
    before = lib.tn_h2d_copy_count()
    for i in list(range(0, 10)) + list(range(500, 520)):
        A.check(lib.tn_assign_from_host(C.byref(dev0), values.data_ptr() + 4 * i, target.data_ptr() + 4 * i, 4))
    doubled = tb.add(target, target)
    assert lib.tn_h2d_copy_count() == before + 2
    want = torch.zeros(1000)
    want[0:10], want[500:520] = values[0:10] * 2, values[500:520] * 2
    assert torch.equal(doubled.cpu(), want)
    A.check(lib.tn_flush_assignments())
