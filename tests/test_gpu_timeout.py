"""A bounded device-side wait that runs out: the kernel returns, the host reads EMA_ERR_TIMEOUT once, the status word
clears, and the library keeps working.  Nothing faults, traps or hangs: a single small thread block waits a few
milliseconds for an mbarrier (or an arrival counter) that nothing ever completes, through the same wait functions as
the tensor-core kernels, with a limit of a thousand polls."""
import ctypes

import numpy as np
import pytest
import torch

from helpers import check_outputs, make_inputs, oracle_fwd_bwd

pytestmark = pytest.mark.gpu

EMA_ERR_TIMEOUT = -5


@pytest.mark.parametrize("mode", [0, 1])
def test_a_wait_that_runs_out_is_reported_and_harmless(mode, ema_lib):
    from ema_b200 import ops
    from ema_b200._lib import EmaB200Error, ptr, stream_ptr
    dev = torch.device("cuda")
    torch.cuda.synchronize()
    assert ema_lib.ema_b200_device_status(1) == 0
    zero = torch.zeros(1, dtype=torch.int32, device=dev)
    rc = ema_lib.ema_b200_selftest_wait(mode, 1000, ptr(zero), stream_ptr(dev))
    assert rc == 0
    torch.cuda.synchronize()                      # the launch returns by itself
    assert ema_lib.ema_b200_device_status(0) == EMA_ERR_TIMEOUT   # reading without clearing keeps it
    assert ema_lib.ema_b200_device_status(1) == EMA_ERR_TIMEOUT
    assert ema_lib.ema_b200_device_status(1) == 0
    assert int(zero.item()) == 0
    # the library still computes correctly afterwards, on both kernel families
    for dtype in (torch.bfloat16, torch.float32):
        x, a, dy, np_in = make_inputs(31 + mode, 2, 384, 2, 128, per_head=True, dtype=dtype)
        f = ops.ema_fwd(x, a, want_tile_states=True, check_status=True)
        r = ops.ema_bwd(x, a, dy, f["tile_states"], check_status=True)
        y_ref, dx_ref, da_ref = oracle_fwd_bwd(np_in)
        check_outputs(dtype, f["y"], y_ref, "y")
        check_outputs(dtype, r["dx"], dx_ref, "dx")
        check_outputs(dtype, r["ddecay"], da_ref, "da", grad_of_decay=True)
    # check_status=True turns a recorded timeout into an exception of the call that reads it
    assert ema_lib.ema_b200_selftest_wait(mode, 500, ptr(zero), stream_ptr(dev)) == 0
    x, a, dy, _ = make_inputs(3, 1, 128, 1, 64, per_head=True, dtype=torch.float32)
    with pytest.raises(EmaB200Error) as err:
        ops.ema_fwd(x, a, check_status=True)
    assert err.value.code == EMA_ERR_TIMEOUT
    assert ema_lib.ema_b200_device_status(1) == 0


def test_selftest_rejects_bad_arguments(ema_lib):
    from ema_b200._lib import ptr, stream_ptr
    dev = torch.device("cuda")
    assert ema_lib.ema_b200_selftest_wait(2, 1000, None, stream_ptr(dev)) == -1
    assert ema_lib.ema_b200_selftest_wait(0, 0, None, stream_ptr(dev)) == -1
    assert ema_lib.ema_b200_selftest_wait(0, (1 << 20) + 1, None, stream_ptr(dev)) == -1
    assert ema_lib.ema_b200_selftest_wait(1, 1000, None, stream_ptr(dev)) == -1
    torch.cuda.synchronize()
    assert ema_lib.ema_b200_device_status(1) == 0
