"""The bounds-checking build (libema_b200_checked.so, -DEMA_BOUNDS_CHECK): every plain global-memory access of the fused
kernels is checked against the address ranges of the call's own buffers; a rejected access is recorded and redirected
to a sink, nothing traps.

The outer test starts a second pytest run of the parity tests of the fused path with that library (EMA_B200_LIB) and
EMA_B200_EXPECT_CHECKED=1, under which a fixture in conftest.py asserts after every test that the checker's status word
is still 0.  The inner tests of this file run only inside that second run: they make the checker reject stores on
purpose - by registering the output tensor as shorter than it is, so that the rejected addresses are memory the test
owns - and check that the stores were redirected and the violation reported."""
import os
import subprocess
import sys

import pytest
import torch

from helpers import make_inputs

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
INNER = os.environ.get("EMA_B200_EXPECT_CHECKED") == "1"
# (not the host pipeline: it keeps calls in flight on several streams, and the checker's table describes one call at a time)
PARITY_FILES = ["tests/test_gpu_fused.py", "tests/test_gpu_tc.py", "tests/test_gpu_aggregates.py",
                "tests/test_gpu_weighted.py", "tests/test_gpu_seqpar_single.py", "tests/test_gpu_fp32_tma.py",
                "tests/test_gpu_guard_zones.py", "tests/test_gpu_fuzz.py", "tests/test_gpu_dropins.py", "tests/test_gpu_stages.py",
                "tests/test_gpu_heads_style.py", "tests/test_gpu_bounds_build.py"]


@pytest.mark.skipif(INNER, reason="this is the run the outer test started")
def test_parity_suite_passes_under_the_bounds_checking_build(ema_lib):
    sys.path.insert(0, os.path.join(ROOT, "triton-kernels_b200"))
    import build as ema_build
    checked = ema_build.build_checked()
    env = dict(os.environ, EMA_B200_LIB=checked, EMA_B200_EXPECT_CHECKED="1")
    r = subprocess.run([sys.executable, "-m", "pytest", *PARITY_FILES, "-x", "-q", "-m", "gpu", "-p", "no:cacheprovider"],
                       cwd=ROOT, env=env, capture_output=True, text=True, timeout=1500)
    tail = "\n".join((r.stdout + r.stderr).splitlines()[-25:])
    assert r.returncode == 0, tail
    assert " passed" in r.stdout and " failed" not in r.stdout, tail


@pytest.mark.skipif(not INNER, reason="runs inside the run the outer test starts with the checking library")
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_checker_rejects_redirects_and_reports(dtype, ema_lib):
    from ema_b200 import ops
    assert ema_lib.ema_b200_bounds_checked() == 1
    b, L, h, d = 2, 200, 2, 20                 # d = 20: rows of 40 or 80 bytes, y leaves by plain stores for both dtypes
    x, a, dy, _ = make_inputs(3, b, L, h, d, per_head=False, dtype=dtype)
    ref = ops.ema_fwd(x, a)["y"]
    assert ema_lib.ema_b200_last_path() != 1   # not the tensor-core kernel (its y leaves by TMA, clipped by the tensor map)
    assert ema_lib.ema_b200_bounds_status(1) == 0
    sentinel = -7.0e4
    y = torch.full_like(ref, sentinel)
    cut = 40                                   # elements of y the registered range leaves out at its end
    assert ema_lib.ema_b200_bounds_shrink_next(cut * y.element_size()) == 0
    ops.ema_fwd(x, a, out=y)
    status = ema_lib.ema_b200_bounds_status(1)
    assert status & 0x400 and (status & 0x3ff) in (9, 10), hex(status)   # the forward's store of y
    assert ema_lib.ema_b200_bounds_status(1) == 0                         # cleared by the read above
    flat, flat_ref = y.reshape(-1), ref.reshape(-1)
    n = flat.numel()
    # a store is rejected when any of its bytes lies in the cut: everything a vector width before the cut arrived,
    # nothing inside the cut was written
    assert torch.equal(flat[:n - cut - 4], flat_ref[:n - cut - 4])
    assert bool((flat[n - cut:] == sentinel).all())
    # the hook is one-shot: the next call is checked against the true extent and passes
    ops.ema_fwd(x, a, out=y)
    assert ema_lib.ema_b200_bounds_status(1) == 0
    assert torch.equal(y, ref)


@pytest.mark.skipif(not INNER, reason="runs inside the run the outer test starts with the checking library")
def test_backward_store_is_checked_too(ema_lib):
    from ema_b200 import ops
    b, L, h, d = 1, 130, 2, 8
    x, a, dy, _ = make_inputs(4, b, L, h, d, per_head=True, dtype=torch.float32)
    f = ops.ema_fwd(x, a, want_tile_states=True)
    ref = ops.ema_bwd(x, a, dy, f["tile_states"])
    assert ema_lib.ema_b200_bounds_status(1) == 0
    dx = torch.full_like(ref["dx"], -7.0e4)
    assert ema_lib.ema_b200_bounds_shrink_next(16 * 4) == 0
    ops.ema_bwd(x, a, dy, f["tile_states"], dx=dx)
    status = ema_lib.ema_b200_bounds_status(1)
    assert status == (0x400 | 61), hex(status)
    assert bool((dx.reshape(-1)[-16:] == -7.0e4).all())
    assert torch.equal(dx.reshape(-1)[:-20], ref["dx"].reshape(-1)[:-20])


def test_normal_build_reports_no_checker(ema_lib):
    if INNER:
        pytest.skip("the checking library is loaded")
    assert ema_lib.ema_b200_bounds_checked() == 0
    assert ema_lib.ema_b200_bounds_status(1) == 0
    assert ema_lib.ema_b200_bounds_shrink_next(16) == -3   # EMA_ERR_UNSUPPORTED


@pytest.mark.skipif(not INNER, reason="runs inside the run the outer test starts with the checking library")
def test_stage_kernels_are_checked_too(ema_lib):
    """A stage call whose output is registered 64 bytes short: the last stores of the cumulative sums are rejected
    (site 321, the chunk-cumsum kernel's output pointer) and everything before them still arrives."""
    from ema_b200 import stages
    A = -torch.rand(2, 200, device="cuda")
    ref = stages.chunk_cumsum(A, 64)
    assert ema_lib.ema_b200_bounds_status(1) == 0
    assert ema_lib.ema_b200_bounds_shrink_next(64) == 0
    cut = stages.chunk_cumsum(A, 64)
    status = ema_lib.ema_b200_bounds_status(1)
    assert status == (0x400 | 321), hex(status)
    assert torch.equal(cut.reshape(-1)[:-16], ref.reshape(-1)[:-16])
    again = stages.chunk_cumsum(A, 64)
    assert ema_lib.ema_b200_bounds_status(1) == 0 and torch.equal(again, ref)
