"""Failure detection on the device path, tested without faulting or hanging a GPU.

The device-side waits of the tensor-core kernels are bounded; what a run-out wait does (abort flag,
error counter, TN_ERROR from the next synchronising call) is exercised by a one-warp kernel that
waits on a barrier nothing completes. Each case runs in a child process so that the error counter
it raises does not leak into other tests' `device_errors() == 0` checks.
"""
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def run_child(body: str) -> None:
    script = "import sys\nsys.path.insert(0, %r)\n" % str(ROOT) + textwrap.dedent(body)
    done = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, timeout=300)
    assert done.returncode == 0, done.stdout + done.stderr
    assert "CHILD_OK" in done.stdout


def test_bounded_wait_runs_out_and_is_reported():
    """The wait gives up after its poll limit: the kernel returns normally, the abort counter rises, and
    the next synchronising call returns TN_ERROR with a message, once. The context stays usable: a
    following op computes the right result and the next synchronise is clean again."""
    run_child("""
        import ctypes as C
        import torch
        import oracle
        from tannic_b200 import _abi as A, ops as tb
        lib = A.lib()
        dev0 = A.DeviceT(0)
        torch.cuda.set_device(0)
        stream = tb.current_stream(torch.empty(1, device="cuda"))
        assert tb.device_errors() == 0
        assert lib.tn_stream_synchronize(stream) == A.SUCCESS
        A.check(lib.tn_selftest_bounded_wait(C.byref(dev0), stream, 4096))
        assert lib.tn_stream_synchronize(stream) == A.ERROR
        assert b"bounded device-side wait" in lib.tn_last_error(), lib.tn_last_error()
        assert tb.device_errors() == 1
        assert lib.tn_stream_synchronize(stream) == A.SUCCESS
        # a copy back to the host reports it too
        A.check(lib.tn_selftest_bounded_wait(C.byref(dev0), stream, 64))
        host = torch.zeros(4, dtype=torch.int32)
        devt = torch.arange(4, dtype=torch.int32, device="cuda")
        assert lib.tn_copy_to_host(C.byref(dev0), devt.data_ptr(), host.data_ptr(), 16) == A.ERROR
        assert host.tolist() == [0, 1, 2, 3]
        a = oracle.fill((64, 128), torch.int32, 70, "uniform", -100, 100)
        b = oracle.fill((64, 1), torch.int32, 71, "uniform", -100, 100)
        assert torch.equal(tb.add(a.cuda(), b.cuda()).cpu(), oracle.binary("add", a, b))
        assert lib.tn_stream_synchronize(stream) == A.SUCCESS
        print("CHILD_OK")
    """)


def test_allocation_failure_is_a_status_not_an_exit():
    """An absurd allocation fails with TN_ERROR and a null address (the reference exits the process,
    src/cuda/exc.cuh:8-16); the next allocation works."""
    run_child("""
        import ctypes as C
        from tannic_b200 import _abi as A
        lib = A.lib()
        dev0 = A.DeviceT(0)
        address = C.c_void_p(1)
        assert lib.tn_allocate(C.byref(dev0), 1 << 60, C.byref(address)) == A.ERROR
        assert not address.value
        assert b"failed" in lib.tn_last_error()
        assert lib.tn_allocate(C.byref(dev0), 1 << 20, C.byref(address)) == A.SUCCESS and address.value
        assert lib.tn_deallocate(C.byref(dev0), address) == A.SUCCESS
        print("CHILD_OK")
    """)
