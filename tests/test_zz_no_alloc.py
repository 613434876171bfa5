"""tn_argsum_fixed_scratch: the row sum for callers that cannot allocate device memory.

Some hosts call this library from a place where asking for device memory is not an option: the
process has already divided all of HBM between its own buffers, or the calling path must avoid
the locks and implicit synchronisation of an allocator. For them the split reduction keeps its
partial sums in a fixed 192 KiB region inside the library. This test calls that entry point
through the C ABI twice in a row (the second call reuses the region the first one dirtied, with
a different shape) and checks each result against tn_argsum on the same input, within the
tolerances of the other parity tests. Collected last so that a run that stops at the first
failure has already run everything else; it also passes alone in a fresh process.
"""
import ctypes as C

import pytest
import torch

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
    g = torch.Generator(device="cuda")
    g.manual_seed(5)
    first = torch.rand((3, 1 << 20), device="cuda", generator=g) * 2 - 1           # float32, long rows, many segments
    second = (torch.rand((40, 70001), device="cuda", generator=g) * 2 - 1).to(torch.bfloat16)  # ragged bf16 rows
    for x, (rtol, atol) in ((first, (1e-4, 1e-5)), (second, (1e-2, 1e-2))):
        got = fixed_sum(x)
        want = tb.sum(x, -1)
        torch.cuda.synchronize()
        assert got.dtype == want.dtype and got.shape == want.shape
        assert close(got, want, rtol, atol)
    ints = torch.randint(-1000, 1000, (7, 300000), dtype=torch.int32, device="cuda", generator=g)
    assert torch.equal(fixed_sum(ints), tb.sum(ints, -1))


def test_limits_are_refused_with_a_message():
    x = torch.zeros((9000, 8), device="cuda")
    with pytest.raises(A.TannicError) as e:
        fixed_sum(x)
    assert e.value.status == A.ERROR and "fixed scratch" in str(e.value)
    y = torch.zeros((8, 16), device="cuda").t()
    with pytest.raises(A.TannicError):
        fixed_sum(y)
