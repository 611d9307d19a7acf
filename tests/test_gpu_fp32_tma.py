"""The fp32 forward has two feeds for the same arithmetic: plain global loads with a register prefetch, and a TMA
ring in shared memory (the default on 16-byte aligned layouts).  Both must give bit-identical results, and the
TMA-fed one must meet the fp32 tolerance against the oracle on its own."""
import numpy as np
import pytest
import torch

from helpers import make_inputs
from oracle import ema_oracle as eo

pytestmark = pytest.mark.gpu

SHAPES = [
    (2, 256, 2, 64),       # the CPU-sized configuration
    (1, 40, 1, 8),         # a fraction of a tile, a fraction of a channel box
    (2, 129, 3, 100),      # ragged in both directions (d a multiple of 4)
    (3, 1111, 2, 192),
    (1, 700, 1, 1024),
    (2, 300, 2, 4),
]


@pytest.fixture(autouse=True)
def _restore_path(ema_lib):
    yield
    ema_lib.ema_b200_set_path(0)


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("per_head", [False, True])
def test_tma_fed_forward_is_bit_identical_to_the_plain_kernel(shape, per_head, ema_lib):
    from ema_b200 import ops
    b, L, h, d = shape
    x, a, _, np_in = make_inputs(40 + L + d, b, L, h, d, per_head=per_head, dtype=torch.float32)
    init = torch.randn(b, h, d, device="cuda")
    kw = dict(chunk=96, want_chunk_states=True, want_tile_states=True, want_final=True, want_log_decay_sum=True,
              init_state=init)
    ema_lib.ema_b200_set_path(0)
    t = ops.ema_fwd(x, a, **kw)
    torch.cuda.synchronize()
    assert ema_lib.ema_b200_last_path() == 2
    ema_lib.ema_b200_set_path(1)
    f = ops.ema_fwd(x, a, **kw)
    torch.cuda.synchronize()
    assert ema_lib.ema_b200_last_path() == 0
    for key in ("y", "chunk_states", "tile_states", "final_state", "log_decay_sum"):
        assert torch.equal(t[key], f[key]), key
    # and against the oracle, without an initial state
    ema_lib.ema_b200_set_path(0)
    y = ops.ema_fwd(x, a)["y"]
    y_ref = eo.fwd(np_in[0], np_in[1])
    assert np.abs(y.cpu().numpy() - y_ref).max() <= 1e-4
    assert ema_lib.ema_b200_device_status(0) == 0


def test_views_the_tma_cannot_describe_take_the_plain_kernel(ema_lib):
    from ema_b200 import ops
    # d = 6: not a multiple of 4 elements
    x, a, _, np_in = make_inputs(7, 2, 200, 2, 6, dtype=torch.float32)
    y = ops.ema_fwd(x, a)["y"]
    torch.cuda.synchronize()
    assert ema_lib.ema_b200_last_path() == 0
    assert np.abs(y.cpu().numpy() - eo.fwd(np_in[0], np_in[1])).max() <= 1e-4
    # a [b, h, L, d] storage viewed as [b, L, h, d]: legal for TMA, strides carried by the tensor map
    xs = torch.randn(2, 2, 260, 64, device="cuda").permute(0, 2, 1, 3)
    a2 = torch.sigmoid(2 + 4 * torch.rand(2, 260, 2, device="cuda"))
    y1 = ops.ema_fwd(xs, a2)["y"]
    torch.cuda.synchronize()
    assert ema_lib.ema_b200_last_path() == 2
    y2 = ops.ema_fwd(xs.contiguous(), a2)["y"]
    assert torch.equal(y1, y2)


def test_weighted_forward_through_both_feeds(ema_lib):
    from ema_b200 import ops
    x, a, _, _ = make_inputs(9, 2, 520, 2, 128, dtype=torch.float32)
    g = torch.Generator(device="cuda").manual_seed(3)
    w = torch.rand(a.shape, generator=g, device="cuda")
    c = torch.randn(a.shape, generator=g, device="cuda")
    ema_lib.ema_b200_set_path(0)
    t = ops.ema_fwd(x, torch.log(a), prescaled_log=True, in_weight=w, out_weight=c, want_final=True)
    torch.cuda.synchronize()
    assert ema_lib.ema_b200_last_path() == 2
    ema_lib.ema_b200_set_path(1)
    f = ops.ema_fwd(x, torch.log(a), prescaled_log=True, in_weight=w, out_weight=c, want_final=True)
    assert torch.equal(t["y"], f["y"]) and torch.equal(t["final_state"], f["final_state"])


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("per_head", [False, True])
@pytest.mark.parametrize("prescaled", [False, True])
def test_tma_fed_backward_is_bit_identical_to_the_plain_kernel(shape, per_head, prescaled, ema_lib):
    from ema_b200 import ops
    from helpers import oracle_fwd_bwd
    b, L, h, d = shape
    x, a, dy, np_in = make_inputs(60 + L + d, b, L, h, d, per_head=per_head, dtype=torch.float32)
    dec = torch.log(a) if prescaled else a
    dfin = torch.randn(b, h, d, device="cuda")
    ema_lib.ema_b200_set_path(1)
    f = ops.ema_fwd(x, dec, want_tile_states=True, prescaled_log=prescaled)
    gp = ops.ema_bwd(x, dec, dy, f["tile_states"], dfinal_state=dfin, want_dinit=True, prescaled_log=prescaled)
    torch.cuda.synchronize()
    assert ema_lib.ema_b200_last_path() == 0
    ema_lib.ema_b200_set_path(0)
    gt = ops.ema_bwd(x, dec, dy, f["tile_states"], dfinal_state=dfin, want_dinit=True, prescaled_log=prescaled)
    torch.cuda.synchronize()
    assert ema_lib.ema_b200_last_path() == 2
    for key in ("dx", "ddecay", "dinit_state"):
        assert torch.equal(gt[key], gp[key]), key
    if not prescaled:
        # and against the oracle, plain problem
        f2 = ops.ema_fwd(x, a, want_tile_states=True)
        g2 = ops.ema_bwd(x, a, dy, f2["tile_states"])
        _, dx_ref, da_ref = oracle_fwd_bwd(np_in)
        assert np.abs(g2["dx"].cpu().numpy() - dx_ref).max() <= 1e-4
        assert np.abs(g2["ddecay"].cpu().numpy() - da_ref).max() <= 1e-4 + 2e-5 * np.abs(da_ref).max()
    assert ema_lib.ema_b200_device_status(0) == 0
