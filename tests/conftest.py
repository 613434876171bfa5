import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def ref_lib():
    """The reference's own CPU kernels (oracle/_ref); tests that need it skip where it was never built."""
    import oracle
    lib = oracle.ref()
    if lib is None:
        pytest.skip("oracle/_ref/libtannic_ref.so not built on this machine")
    return lib
