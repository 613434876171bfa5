"""The reference's own CUDA test files (tests/cuda/test-cuda-*.cpp of the reference), compiled
UNMODIFIED together with its unmodified front-end against this backend
(tannic_b200/dropin: cuda_binding.cpp + a minimal gtest stand-in), run here as executables.

They are built where the reference tree exists (`make -C tannic_b200/dropin`, also done by
`__graft_entry__.build()`); the binaries travel to the GPU machine. A test is skipped when its
binary was never built. Exit code = number of failed gtest cases."""
import subprocess
from pathlib import Path

import pytest

BUILD = Path(__file__).resolve().parent.parent / "tannic_b200" / "dropin" / "_build"
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
