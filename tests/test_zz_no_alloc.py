"""ema_b200_bwd_static_scratch: the backward that uses the library's built-in scratch array instead of a
caller's workspace.  Called through the C interface (ctypes) and compared with ema_b200_bwd on the same
inputs, two calls in a row; the file name sorts last so that it also runs after every other GPU test."""
import ctypes

import numpy as np
import pytest
import torch

from helpers import BF16_REL, FP32_ATOL, make_inputs

pytestmark = pytest.mark.gpu


CASES = [
    # dtype, per-head decay, shape
    (torch.bfloat16, True, (4, 1024, 2, 256)),    # tensor-core kernels
    (torch.bfloat16, False, (1, 300, 2, 64)),     # per-step decay
    (torch.float32, True, (2, 515, 3, 40)),       # CUDA-core kernels, ragged
    (torch.float32, False, (1, 257, 2, 24)),
]


@pytest.mark.parametrize("dtype,per_head,shape", CASES)
def test_static_scratch_backward_matches_workspace_backward(dtype, per_head, shape, ema_lib):
    from ema_b200 import ops
    from ema_b200._lib import ptr, stream_ptr
    b, L, h, d = shape
    x, a, dy, _ = make_inputs(4242, b, L, h, d, per_head=per_head, dtype=dtype)
    fwd = ops.ema_fwd(x, a, want_tile_states=True)
    ref = ops.ema_bwd(x, a, dy, fwd["tile_states"])
    torch.cuda.synchronize()
    p = ops._problem(x, a, ref["dx"], dy=dy)
    assert ema_lib.ema_b200_bwd_workspace_bytes(ctypes.byref(p)) <= ema_lib.ema_b200_static_scratch_limit()

    dx_ref = ref["dx"].float().cpu().numpy()
    da_ref = ref["ddecay"].float().cpu().numpy()
    for call in range(2):
        # fresh outputs filled with a sentinel; a different dy scale per call, so that a stale result shows
        scale = 1.0 + call
        dy_c = (dy.float() * scale).to(dtype)
        dx = torch.full_like(x, float("nan"))
        da = torch.full_like(a, float("nan"))
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        rc = ema_lib.ema_b200_bwd_static_scratch(ctypes.byref(p), ptr(x), ptr(a), ptr(dy_c), ptr(fwd["tile_states"]),
                                                 ptr(dx), ptr(da), stream_ptr(x.device))
        assert rc == 0, ema_lib.ema_b200_error_string(rc).decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        got_dx = dx.float().cpu().numpy() / scale
        got_da = da.float().cpu().numpy() / scale
        # the same kernels ran on the same inputs (dy scaled by a power of two): the test tolerance is generous
        if dtype == torch.float32:
            assert np.abs(got_dx - dx_ref).max() <= FP32_ATOL
            assert np.abs(got_da - da_ref).max() <= FP32_ATOL + 2e-5 * np.abs(da_ref).max()
        else:
            assert np.abs(got_dx - dx_ref).max() <= BF16_REL * np.abs(dx_ref).max()
            assert np.abs(got_da - da_ref).max() <= BF16_REL * np.abs(da_ref).max()
    assert ema_lib.ema_b200_device_status(0) == 0


def test_python_wrapper_and_size_limit(ema_lib):
    from ema_b200 import ops
    from ema_b200._lib import EmaB200Error
    x, a, dy, _ = make_inputs(7, 2, 384, 2, 128, per_head=True, dtype=torch.bfloat16)
    fwd = ops.ema_fwd(x, a, want_tile_states=True)
    ref = ops.ema_bwd(x, a, dy, fwd["tile_states"])
    dx, da = torch.empty_like(x), torch.empty_like(a)
    ops.ema_bwd_static_scratch(x, a, dy, fwd["tile_states"], dx, da)
    torch.cuda.synchronize()
    assert torch.equal(dx, ref["dx"])
    assert torch.equal(da, ref["ddecay"])

    # a per-step decay at this size needs 32 rows * 32 channel slices * 32 tiles * 128 floats = 16 MiB > the 8 MiB array:
    # refused, nothing runs
    assert ops.static_scratch_limit() == 8 << 20
    b, L, h, d = 2, 4096, 16, 512
    xs = torch.zeros((b, L, h, d), dtype=torch.bfloat16, device="cuda")
    as_ = torch.full((b, L, h), 0.9, dtype=torch.float32, device="cuda")
    ts = torch.zeros((b * h, L // 128, d), dtype=torch.float32, device="cuda")
    dxs = torch.full_like(xs, 3.0)
    das = torch.full_like(as_, 3.0)
    p = ops._problem(xs, as_, dxs, dy=xs)
    assert ema_lib.ema_b200_bwd_workspace_bytes(ctypes.byref(p)) > ops.static_scratch_limit()
    with pytest.raises(EmaB200Error) as err:
        ops.ema_bwd_static_scratch(xs, as_, xs, ts, dxs, das)
    assert err.value.code == -7 and "scratch" in str(err.value)
    torch.cuda.synchronize()
    assert bool((dxs == 3.0).all()) and bool((das == 3.0).all())
