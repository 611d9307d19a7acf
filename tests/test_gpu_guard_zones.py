"""Out-of-bounds writes, looked for with guard zones: every buffer a fused call writes (y, dx, the saved tile states, the
final state, the summed log decay, dinit, the decay gradient, the forward scratch and the backward workspace) is a
view into the middle of a larger allocation whose margins hold a sentinel; after the call the margins must be
untouched.  Small and awkward shapes (ragged L and d, one step, one channel, a half-filled channel tile), both kernel
families, all three schedules of the tensor-core kernels, both decay modes.  Nothing here can fault: a stray write
lands in memory the test owns."""
import ctypes

import pytest
import torch

from helpers import make_inputs

pytestmark = pytest.mark.gpu

GUARD = 4096          # elements of margin on either side
SENTINEL = -7.0e4     # exactly representable in bf16 and fp32


class Guarded:
    """A tensor of `shape` inside a flat allocation with a sentinel-filled margin before and after it."""

    def __init__(self, shape, dtype):
        n = 1
        for s in shape:
            n *= s
        self.flat = torch.full((n + 2 * GUARD,), SENTINEL, dtype=dtype, device="cuda")
        self.view = self.flat[GUARD:GUARD + n].view(shape)
        self.n = n

    def intact(self):
        return bool((self.flat[:GUARD] == SENTINEL).all()) and bool((self.flat[GUARD + self.n:] == SENTINEL).all())


SHAPES = [(1, 1, 1, 8), (2, 127, 2, 8), (1, 129, 3, 72), (2, 300, 2, 64), (1, 513, 1, 136), (3, 260, 2, 256), (1, 1000, 2, 24),
          (2, 77, 1, 1), (1, 2049, 2, 200)]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("per_head", [False, True])
@pytest.mark.parametrize("split", [0, 1, 2])
def test_no_call_writes_outside_its_buffers(shape, dtype, per_head, split, ema_lib):
    from ema_b200 import ops
    if dtype == torch.float32 and split != 1:
        pytest.skip("the schedules only concern the bf16 kernels")
    b, L, h, d = shape
    before = ema_lib.ema_b200_set_split(split)
    try:
        x, a, dy, _ = make_inputs(5 + L, b, L, h, d, per_head=per_head, dtype=dtype)
        ts_steps, nt = ops.n_tiles_of(x, a)
        p = ops._problem(x, a, x, dy=dy)
        y = Guarded((b, L, h, d), dtype)
        dx = Guarded((b, L, h, d), dtype)
        ts = Guarded((b * h, nt, d), torch.float32)
        fin = Guarded((b, h, d), torch.float32)
        lds = Guarded((b, h), torch.float32)
        dinit = Guarded((b, h, d), torch.float32)
        da = Guarded(tuple(a.shape), torch.float32)
        fws = Guarded((max(1, (ema_lib.ema_b200_fwd_workspace_bytes(ctypes.byref(p)) + 3) // 4),), torch.float32)
        bws = Guarded((max(1, (ema_lib.ema_b200_bwd_workspace_bytes(ctypes.byref(p)) + 3) // 4),), torch.float32)
        # the scratch views start 16-byte aligned (GUARD elements of 4 bytes)
        ops.ema_fwd(x, a, out=y.view, tile_states=ts.view, final_out=fin.view, workspace=fws.view)
        ops.ema_fwd(x, a, out=y.view, tile_states=ts.view, final_out=fin.view, log_decay_sum_out=lds.view,
                    workspace=fws.view)
        ops.ema_bwd(x, a, dy, ts.view, dx=dx.view, ddecay=da.view, workspace=bws.view, dinit_out=dinit.view)
        torch.cuda.synchronize()
        for g, what in ((y, "y"), (dx, "dx"), (ts, "tile states"), (fin, "final state"), (lds, "log decay sum"),
                        (dinit, "dinit"), (da, "decay gradient"), (fws, "forward scratch"), (bws, "backward workspace")):
            assert g.intact(), f"{what}: a write landed outside the buffer"
        # and the outputs themselves were all written
        assert bool(torch.isfinite(y.view.float()).all()) and bool((y.view != SENTINEL).any() or L * d == 0)
        assert bool(torch.isfinite(dx.view.float()).all())
    finally:
        ema_lib.ema_b200_set_split(before)
    assert ema_lib.ema_b200_device_status(1) == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_weighted_calls_and_the_fold_stay_inside_their_buffers(dtype, ema_lib):
    from ema_b200 import ops
    b, L, h, d = 2, 261, 2, 72
    x, a, dy, _ = make_inputs(9, b, L, h, d, per_head=False, dtype=dtype)
    w = torch.rand((b, L, h), device="cuda") + 0.1
    c = torch.randn((b, L, h), device="cuda")
    f = ops.ema_fwd(x, a, want_tile_states=True, in_weight=w, out_weight=c)
    r = ops.ema_bwd_weighted(x, a, dy, f["tile_states"], in_weight=w, out_weight=c, want_dinit=True)
    torch.cuda.synchronize()
    assert all(bool(torch.isfinite(t.float()).all()) for t in (f["y"], r["dx"], r["ddecay"], r["din_weight"], r["dout_weight"]))
    rows = b * h
    recs = torch.randn((3, rows * d + rows), device="cuda")
    recs[:, rows * d:] = -torch.rand((3, rows), device="cuda")
    out = Guarded((rows, d), torch.float32)
    ops.fold_records(recs, 2, rows, d, out=out.view)
    ops.fold_records(recs, 0, rows, d, reverse=True, out=out.view)
    torch.cuda.synchronize()
    assert out.intact()
