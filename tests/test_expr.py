"""The lazy expression layer: trees become `tn_eltwise_program` node lists (CPU: structure only; gpu: results)."""
import pytest
import torch

import oracle
from tannic_b200 import _abi as A
from tannic_b200 import expr as E


def test_config2_expression_compiles_to_the_benchmark_program():
    x, y = torch.zeros(4, 8, dtype=torch.float16), torch.zeros(1, 8, dtype=torch.float16)
    X, Y = E.lazy(x), E.lazy(y)
    inputs, nodes = (E.log(X) + Y * Y - E.exp(X)).compile(require_device=False)
    assert [t.data_ptr() for t in inputs] == [x.data_ptr(), y.data_ptr()]
    assert [n[:3] for n in nodes] == [(A.OP_LOG, 0, 0), (A.OP_MUL, 1, 1), (A.OP_ADD, 4, 5), (A.OP_EXP, 0, 0), (A.OP_SUB, 6, 7)]


def test_common_subexpressions_are_merged_and_scalars_scale():
    x = torch.zeros(3, dtype=torch.float32)
    X = E.lazy(x)
    sq = X * X
    inputs, nodes = ((sq + sq) * 0.5).compile(require_device=False)
    assert len(inputs) == 1
    assert [n[:3] for n in nodes] == [(A.OP_MUL, 0, 0), (A.OP_ADD, 4, 4), (A.OP_SCALE, 5, 5)]
    assert nodes[-1][3] == 0.5
    _, nodes = E.rsqrt(X, 1e-5).compile(require_device=False)
    assert nodes == [(A.OP_RSQRT, 0, 0, 1e-5)]


def test_trees_that_do_not_fit_are_not_fused():
    f32, f16 = torch.zeros(3, dtype=torch.float32), torch.zeros(3, dtype=torch.float16)
    assert (E.lazy(f32) + E.lazy(f16)).compile(require_device=False) is None          # two dtypes
    assert (E.lazy(torch.zeros(3, dtype=torch.int32)) + E.lazy(torch.zeros(3, dtype=torch.int32))).compile(require_device=False) is None
    five = [E.lazy(torch.zeros(3)) for _ in range(5)]
    assert (five[0] + five[1] + five[2] + five[3] + five[4]).compile(require_device=False) is None  # five tensors
    e = E.lazy(f32)
    for _ in range(17):
        e = E.exp(e)
    assert e.compile(require_device=False) is None                                      # seventeen nodes
    assert (E.lazy(f32) + E.lazy(f32)).compile() is None                                # host tensors
    with pytest.raises(TypeError):
        E.lazy(f32) + 1.0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_fused_and_node_by_node_agree_with_the_oracle(dtype):
    x = oracle.fill((96, 200), dtype, 1, "uniform", 0.1, 4.0)
    y = oracle.fill((1, 200), dtype, 2, "uniform", -2.0, 2.0)
    want = oracle.binary("sub", oracle.binary("add", oracle.unary("log", x), oracle.binary("mul", y, y)), oracle.unary("exp", x))
    X, Y = E.lazy(x.cuda()), E.lazy(y.cuda())
    tree = E.log(X) + Y * Y - E.exp(X)
    assert tree.compile() is not None
    tol = 1e-2 if dtype != torch.float32 else 1e-4
    fused = tree.forward().cpu()
    chain = tree._eval({}).cpu()
    for got in (fused, chain):
        assert got.dtype == dtype and torch.allclose(got.double(), want.double(), rtol=tol, atol=tol)
    # a tree outside the compiled shapes takes the interpreter; a mixed-dtype tree is evaluated node by node
    other = E.tanh(X * 0.5) * Y + E.sqrt(X)
    w = oracle.binary("add", oracle.binary("mul", oracle.unary("tanh", oracle.scale(x, 0.5)), y), oracle.unary("sqrt", x))
    assert torch.allclose(other.forward().cpu().double(), w.double(), rtol=tol, atol=tol)
    wider = torch.float64 if dtype == torch.float32 else torch.float32
    z = oracle.fill((96, 200), wider, 3, "uniform", -1, 1)
    mixed = X + E.lazy(z.cuda())
    assert mixed.compile() is None
    assert torch.allclose(mixed.forward().cpu().double(), oracle.binary("add", x, z).double(), rtol=tol, atol=tol)
