"""tannic_b200 — B200 (sm_100a) device backend for Tannic's operator core.

`tannic_b200._abi` is the ctypes view of the C ABI (include/tannic_b200.h); `tannic_b200.ops`
mirrors the reference's operator front-end over torch CUDA tensors. The CUDA library is built
in-tree by `python -m tannic_b200.build`; nothing here falls back to a CPU implementation.
"""
from . import _abi  # noqa: F401

__all__ = ["_abi", "ops", "build"]


def __getattr__(name):
    if name == "ops":
        import importlib
        return importlib.import_module(".ops", __name__)
    if name == "build":
        import importlib
        return importlib.import_module(".build", __name__)
    raise AttributeError(name)
