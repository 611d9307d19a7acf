"""Host-resident problems streamed through the GPU in batch slices (ema_b200.host): the result must equal
the one-shot device computation bit for bit (same kernels, rows are independent) and match the oracle."""
import numpy as np
import pytest
import torch

from helpers import check_outputs, make_inputs, oracle_fwd_bwd

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("per_head", [False, True])
@pytest.mark.parametrize("slices,depth", [(1, 1), (3, 2), (8, 3)])
def test_host_pipeline_matches_device_and_oracle(dtype, per_head, slices, depth, ema_lib):
    import ema_b200
    from ema_b200 import ops
    b, L, h, d = 5, 300, 2, 64
    x, a, dy, np_in = make_inputs(321, b, L, h, d, per_head=per_head, dtype=dtype)
    hx, ha, hdy = x.cpu().pin_memory(), a.cpu().pin_memory(), dy.cpu().pin_memory()
    hy, hdx, hda = torch.empty_like(hx).pin_memory(), torch.empty_like(hx).pin_memory(), torch.empty_like(ha).pin_memory()
    pipe = ema_b200.HostPipeline((b, L, h, d), dtype, per_head=per_head, slices=slices, depth=depth)
    for _ in range(2):     # a second run reuses every buffer and event
        hy.fill_(float("nan")); hdx.fill_(float("nan")); hda.fill_(float("nan"))
        pipe.run(hx, ha, hdy, hy, hdx, hda)
        fwd = ops.ema_fwd(x, a, want_tile_states=True)
        bwd = ops.ema_bwd(x, a, dy, fwd["tile_states"])
        torch.cuda.synchronize()
        assert torch.equal(hy, fwd["y"].cpu())
        assert torch.equal(hdx, bwd["dx"].cpu())
        if per_head:   # summed per slice, then over slices: a different order than the one-shot reduction
            ref = bwd["ddecay"].cpu().numpy()
            assert np.abs(hda.numpy() - ref).max() <= 1e-4 * max(1.0, np.abs(ref).max())
        else:
            assert torch.equal(hda, bwd["ddecay"].cpu())
    y_ref, dx_ref, da_ref = oracle_fwd_bwd(np_in)
    check_outputs(dtype, hy, y_ref, "y")
    check_outputs(dtype, hdx, dx_ref, "dx")
    check_outputs(dtype, hda, da_ref, "da", grad_of_decay=True)
    assert pipe.n_launches == 3 * min(slices, b)   # per slice: forward scan, backward scan, decay-gradient reduction


def test_one_shot_form_and_argument_checks(ema_lib):
    import ema_b200
    x, a, dy, np_in = make_inputs(9, 2, 130, 1, 24, per_head=True, dtype=torch.float32)
    y, dx, da = ema_b200.ema_fwd_bwd_host(x.cpu(), a.cpu(), dy.cpu(), slices=2)
    y_ref, dx_ref, da_ref = oracle_fwd_bwd(np_in)
    check_outputs(torch.float32, y, y_ref, "y")
    check_outputs(torch.float32, dx, dx_ref, "dx")
    check_outputs(torch.float32, da, da_ref, "da", grad_of_decay=True)
    pipe = ema_b200.HostPipeline((2, 130, 1, 24), torch.float32, per_head=True)
    with pytest.raises(ValueError):
        pipe.run(x, a.cpu(), dy.cpu(), y, dx, da)          # x on the device
    with pytest.raises(ValueError):
        pipe.run(x.cpu(), torch.zeros(3), dy.cpu(), y, dx, da)   # wrong decay shape
