"""The reference's own CUDA test files (tests/cuda/test-cuda-*.cpp of the reference), compiled
UNMODIFIED together with its unmodified front-end against this backend
(tannic_b200/dropin/cuda_binding.cpp; tests/dropin: Makefile + a minimal gtest stand-in), run here
as executables, once against the plain drop-in library and, for the elementwise suites, once more
against the fused-by-default header overlay.

They are built where the reference tree exists (`make -C tannic_b200/dropin` then
`make -C tests/dropin`, both done by `__graft_entry__.build()`); the binaries travel to the GPU
machine. A test is skipped when its binary was never built. Exit code = number of failed gtest cases."""
import subprocess
from pathlib import Path

import pytest

BUILD = Path(__file__).resolve().parent / "dropin" / "_build"
SUITES = ["allocations", "complex", "concat", "convolutions", "functions", "indexing", "matmul", "operations", "outer",
          "reductions", "repeats"]


@pytest.mark.gpu
@pytest.mark.parametrize("suite", SUITES)
def test_reference_cuda_suite_passes_on_this_backend(suite):
    exe = BUILD / f"test-cuda-{suite}"
    if not exe.exists():
        pytest.skip(f"{exe.name} not built (needs the reference tree at build time)")
    res = subprocess.run([str(exe)], capture_output=True, text=True, timeout=600)
    tail = "\n".join((res.stdout + res.stderr).splitlines()[-25:])
    assert res.returncode == 0, f"{res.returncode} failing case(s):\n{tail}"
    assert "[ RUN      ]" in res.stdout


@pytest.mark.gpu
def test_reference_expression_templates_evaluate_as_one_kernel():
    """tannic_b200/dropin/fused.hpp walks the reference's Binary / Unary / Function templates and emits one
    `tn_eltwise_program` call; its own test compares that with the expression's node-by-node forward() and
    counts the launches."""
    exe = BUILD / "test-fused-expression"
    if not exe.exists():
        pytest.skip(f"{exe.name} not built (needs the reference tree at build time)")
    res = subprocess.run([str(exe)], capture_output=True, text=True, timeout=600)
    tail = "\n".join((res.stdout + res.stderr).splitlines()[-25:])
    assert res.returncode == 0, f"{res.returncode} failing case(s):\n{tail}"
    assert "[ RUN      ]" in res.stdout


@pytest.mark.gpu
@pytest.mark.parametrize("suite", ["operations", "functions"])
def test_reference_suites_pass_with_fusion_as_the_default(suite):
    """The reference's operations / functions suites, unmodified, compiled against the header overlay
    (tannic_b200/dropin/make_overlay.py, -DTANNIC_B200_FUSE): every multi-node expression in them now
    evaluates as one kernel and the suites' own expectations still hold."""
    exe = BUILD / f"fused-test-cuda-{suite}"
    if not exe.exists():
        pytest.skip(f"{exe.name} not built (needs the reference tree at build time)")
    res = subprocess.run([str(exe)], capture_output=True, text=True, timeout=600)
    tail = "\n".join((res.stdout + res.stderr).splitlines()[-25:])
    assert res.returncode == 0, f"{res.returncode} failing case(s):\n{tail}"
    assert "[ RUN      ]" in res.stdout


@pytest.mark.gpu
def test_plain_assignment_is_one_launch_under_the_overlay():
    """tests/dropin/test-fused-default.cpp: `Tensor Z = log(X) + Y * Y - exp(X);` with no helper is one
    launch, values equal to the host evaluation; trees that do not fit fall back piecewise."""
    exe = BUILD / "test-fused-default"
    if not exe.exists():
        pytest.skip(f"{exe.name} not built (needs the reference tree at build time)")
    res = subprocess.run([str(exe)], capture_output=True, text=True, timeout=600)
    tail = "\n".join((res.stdout + res.stderr).splitlines()[-25:])
    assert res.returncode == 0, f"{res.returncode} failing case(s):\n{tail}"
    assert "[ RUN      ]" in res.stdout
