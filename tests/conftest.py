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


@pytest.fixture(autouse=True)
def _bounds_word_stays_clear(request):
    """Inside the run that tests/test_gpu_bounds_build.py starts with the bounds-checking library: after every test the
    checker's status word must still be 0 (no access outside the call's buffers)."""
    yield
    if os.environ.get("EMA_B200_EXPECT_CHECKED") != "1" or request.node.get_closest_marker("gpu") is None:
        return
    from ema_b200 import _lib
    lib = _lib.lib()
    assert lib.ema_b200_bounds_checked() == 1, "EMA_B200_LIB does not point at the bounds-checking build"
    status = lib.ema_b200_bounds_status(1)
    assert status == 0, f"access outside the call's buffers, site {status & 0x3ff}"
