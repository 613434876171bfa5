"""tn_argsum_fixed_scratch: the row sum for callers that cannot allocate device memory.

Some hosts call this library from a place where asking for device memory is not an option: the
process has already divided all of HBM between its own buffers, or the calling path must avoid
the locks and implicit synchronisation of an allocator. For them the split reduction keeps its
partial sums in a fixed 192 KiB region inside the library. This test calls that entry point
through the C ABI twice in a row (the second call reuses the region the first one dirtied, with
a different shape) and checks each result against tn_argsum on the same input and against the
oracle's sum, within the tolerances of the other parity tests. Collected last so that a run that stops at the first
failure has already run everything else; it also passes alone in a fresh process.
"""
import ctypes as C

import pytest
import torch

import oracle
from tannic_b200 import _abi as A
from tannic_b200 import ops as tb

pytestmark = pytest.mark.gpu


def fixed_sum(x):
    out = torch.empty(x.shape[:-1], dtype=x.dtype, device=x.device)
    dx, dd = tb.desc(x), tb.desc(out)
    A.check(A.lib().tn_argsum_fixed_scratch(C.byref(dx), C.byref(dd), tb.current_stream(x), C.c_uint8(x.dim() - 1)))
    return out


def close(got, want, rtol, atol):
    g, w = got.double().cpu(), want.double().cpu()
    return bool(((g - w).abs() <= atol + rtol * w.abs()).all())


def test_two_calls_in_a_row_match_tn_argsum():
    first = oracle.fill((3, 1 << 20), torch.float32, 5, "uniform", -1.0, 1.0)              # long rows, many segments
    second = oracle.fill((40, 70001), torch.bfloat16, 6, "uniform", -1.0, 1.0)             # ragged bf16 rows
    for host, (rtol, atol) in ((first, (1e-4, 1e-5)), (second, (1e-2, 1e-2))):
        x = host.cuda()
        got = fixed_sum(x)
        want = tb.sum(x, -1)
        torch.cuda.synchronize()
        assert got.dtype == want.dtype and got.shape == want.shape
        assert close(got, want, rtol, atol)
        # and against the checker: the reference's float-accumulating sum of the same values
        assert close(got, oracle.reduce("sum", host, -1, acc=oracle.ACC_WIDE), rtol, atol if host.dtype != torch.float32 else 1e-3)
    ints = oracle.fill((7, 300000), torch.int32, 7, "uniform", -1000, 1000)
    got = fixed_sum(ints.cuda())
    assert torch.equal(got, tb.sum(ints.cuda(), -1))
    assert torch.equal(got.cpu(), oracle.reduce("sum", ints, -1, acc=oracle.ACC_WIDE))


def test_zero_length_rows_sum_to_zero():
    """An empty last axis: every sum is zero, as tn_argsum gives; the result buffer is written."""
    x = torch.empty((5, 0), dtype=torch.float32, device="cuda")
    out = torch.full((5,), 7.0, device="cuda")
    dx, dd = tb.desc(x), tb.desc(out)
    A.check(A.lib().tn_argsum_fixed_scratch(C.byref(dx), C.byref(dd), tb.current_stream(x), C.c_uint8(1)))
    assert torch.equal(out.cpu(), torch.zeros(5)) and torch.equal(tb.sum(x, -1).cpu(), torch.zeros(5))


def test_limits_are_refused_with_a_message():
    x = torch.zeros((9000, 8), device="cuda")  # float32: 24-byte partials, room for 8192 rows
    with pytest.raises(A.TannicError) as e:
        fixed_sum(x)
    assert e.value.status == A.ERROR and "fixed scratch" in str(e.value) and "8192" in str(e.value)
    assert torch.equal(fixed_sum(torch.ones((9000, 8), dtype=torch.bfloat16, device="cuda")).cpu(), torch.full((9000,), 8.0, dtype=torch.bfloat16))
    with pytest.raises(A.TannicError) as e:  # 16-bit sources: 16-byte partials, room for 12288 rows
        fixed_sum(torch.zeros((12289, 8), dtype=torch.float16, device="cuda"))
    assert "12288" in str(e.value)
    y = torch.zeros((8, 16), device="cuda").t()
    with pytest.raises(A.TannicError):
        fixed_sum(y)
