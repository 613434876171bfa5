"""Run-time instantiated element-wise programs (tn_eltwise_program on a node list that no ahead-of-time
program covers): the compiled kernel must agree bit for bit with the in-kernel interpreter and, through
it, with the oracle's node-by-node chain; compilations are counted and cached."""
import pytest
import torch

import oracle
from tannic_b200 import _abi as A
from tannic_b200 import ops as tb

pytestmark = pytest.mark.gpu

HALVES = [torch.float16, torch.bfloat16]


def dev(t):
    return t.cuda()


def gen(shape, dtype, seed, lo, hi):
    return oracle.fill(shape, dtype, seed, "uniform", lo, hi)


@pytest.fixture(autouse=True)
def default_mode_afterwards():
    yield
    tb.program_jit(1)


def both_ways(inputs, nodes):
    """The same program through the interpreter and through the run-time compiler."""
    tb.program_jit(0)
    interpreted = tb.program(inputs, nodes)
    tb.program_jit(2)
    before = tb.program_jit_stats()
    compiled = tb.program(inputs, nodes)
    after = tb.program_jit_stats()
    assert after["available"], "NVRTC or its headers were not found: " + after["log"]
    assert after["failed"] == before["failed"], after["log"]
    torch.cuda.synchronize()
    return interpreted, compiled, after["compiled"] - before["compiled"]


TANH_NODES = [(A.OP_MUL, 0, 1), (A.OP_ADD, 4, 2), (A.OP_TANH, 5, 5), (A.OP_SCALE, 6, 6, 0.5), (A.OP_RSQRT, 0, 0, 1e-3), (A.OP_SUB, 7, 8)]


@pytest.mark.parametrize("dtype", HALVES + [torch.float32])
def test_compiled_program_equals_interpreter_and_oracle(dtype):
    x, w, b = gen((130, 264), dtype, 100, 0.2, 3.0), gen((130, 264), dtype, 101, -2.0, 2.0), gen((264,), dtype, 102, -1.0, 1.0)
    interpreted, compiled, fresh = both_ways([dev(x), dev(w), dev(b)], TANH_NODES)
    assert fresh <= 1
    assert torch.equal(interpreted.view(torch.uint8), compiled.view(torch.uint8))
    O, B, U = oracle, oracle.binary, oracle.unary
    want = B("sub", O.scale(U("tanh", B("add", B("mul", x, w), b)), 0.5), U("rsqrt", x, eps=1e-3))
    g, t = compiled.double().cpu(), want.double()
    tol = 2e-2 if dtype != torch.float32 else 1e-5
    assert bool(((g - t).abs() <= tol + tol * t.abs()).all())
    assert tb.device_errors() == 0


def test_compilation_is_cached_and_immediates_are_arguments():
    x, w = dev(gen((64, 512), torch.float16, 110, 0.5, 2.0)), dev(gen((64, 512), torch.float16, 111, -1.0, 1.0))
    nodes = [(A.OP_SUB, 0, 1), (A.OP_SCALE, 4, 4, 0.25), (A.OP_ABS, 5, 5), (A.OP_SQRT, 6, 6)]
    _, first, _ = both_ways([x, w], nodes)
    before = tb.program_jit_stats()["compiled"]
    launches = tb.launch_count()
    again = tb.program([x, w], nodes)
    other_factor = tb.program([x, w], [(A.OP_SUB, 0, 1), (A.OP_SCALE, 4, 4, 4.0), (A.OP_ABS, 5, 5), (A.OP_SQRT, 6, 6)])
    assert tb.program_jit_stats()["compiled"] == before, "a second call and another immediate reuse the compiled kernel"
    assert tb.launch_count() - launches == 2
    assert torch.equal(again, first)
    want = oracle.unary("sqrt", oracle.unary("abs", oracle.scale(oracle.binary("sub", x.cpu(), w.cpu()), 4.0)))
    assert torch.equal(other_factor.cpu().view(torch.int16), want.view(torch.int16))


def test_column_broadcast_operand():
    # a column-broadcast input selects the kernel variant that branches on the operand kind
    x, col = gen((130, 264), torch.bfloat16, 120, 0.2, 3.0), gen((130, 1), torch.bfloat16, 121, 0.5, 1.5)
    nodes = [(A.OP_MUL, 0, 1), (A.OP_SUB, 4, 0), (A.OP_ABS, 5, 5)]
    interpreted, compiled, _ = both_ways([dev(x), dev(col)], nodes)
    assert torch.equal(interpreted.view(torch.int16), compiled.view(torch.int16))
    want = oracle.unary("abs", oracle.binary("sub", oracle.binary("mul", x, col), x))
    assert torch.equal(compiled.cpu().view(torch.int16), want.view(torch.int16))


def test_small_results_are_interpreted_by_default():
    x, w = dev(gen((16, 64), torch.float16, 130, 0.5, 2.0)), dev(gen((16, 64), torch.float16, 131, -1.0, 1.0))
    tb.program_jit(1)
    before = tb.program_jit_stats()["compiled"]
    tb.program([x, w], [(A.OP_ADD, 0, 1), (A.OP_COS, 4, 4), (A.OP_MUL, 5, 0)])
    assert tb.program_jit_stats()["compiled"] == before
    with pytest.raises(A.TannicError):
        tb.program_jit(3)


def test_disk_cache_between_processes(tmp_path):
    """With TN_PROGRAM_JIT_CACHE set, a second process loads the image the first one compiled."""
    import json
    import os
    import subprocess
    import sys

    script = (
        "import json, torch, oracle\n"
        "from tannic_b200 import _abi as A, ops as tb\n"
        "x = oracle.fill((64, 512), torch.float16, 140, 'uniform', 0.5, 2.0).cuda()\n"
        "w = oracle.fill((64, 512), torch.float16, 141, 'uniform', -1.0, 1.0).cuda()\n"
        "tb.program_jit(2)\n"
        "z = tb.program([x, w], [(A.OP_ADD, 0, 1), (A.OP_SINH, 4, 4), (A.OP_MUL, 5, 1)])\n"
        "torch.cuda.synchronize()\n"
        "s = tb.program_jit_stats(); s['sum'] = float(z.float().sum()); print(json.dumps(s))\n"
    )
    env = dict(os.environ, TN_PROGRAM_JIT_CACHE=str(tmp_path), PYTHONPATH=os.pathsep.join(sys.path))
    runs = []
    for _ in range(2):
        done = subprocess.run([sys.executable, "-c", script], env=env, capture_output=True, text=True, timeout=300)
        assert done.returncode == 0, done.stderr[-2000:]
        runs.append(json.loads(done.stdout.strip().splitlines()[-1]))
    assert runs[0]["compiled"] == 1 and runs[0]["from_disk"] == 0 and runs[0]["failed"] == 0
    assert runs[1]["compiled"] == 0 and runs[1]["from_disk"] == 1 and runs[1]["failed"] == 0
    assert runs[0]["sum"] == runs[1]["sum"]
    assert len(list(tmp_path.glob("tnjit_*.bin"))) == 1
