import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (os.path.join(ROOT, "triton-kernels_b200"), ROOT, os.path.join(ROOT, "tests", "golden"),
          os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with -m gpu)")


@pytest.fixture(scope="session")
def ema_lib():
    """The built CUDA library (compiled on first use; nvcc cross-compiles without a GPU)."""
    sys.path.insert(0, os.path.join(ROOT, "triton-kernels_b200"))
    import build as ema_build
    ema_build.build()
    from ema_b200 import _lib
    return _lib.lib()


@pytest.fixture(scope="session")
def golden_dir():
    return os.path.join(ROOT, "tests", "golden")
