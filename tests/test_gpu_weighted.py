"""Forward scan with per-step weights folded into the pass (ema_b200_fwd_weighted):

    s_t = a_t s_{t-1} + w_t x_t ,     y_t = c_t s_t

against the CPU oracle run on the explicitly weighted input (u = w x in fp32, pre-scaled convention) and scaled
afterwards.  This is what the heads-style entry point (kernels/ema_combined.py of the reference) computes with
w = dt' B and c = C for state size 1.  Both kernel families, either weight alone, states unweighted.
"""
import numpy as np
import pytest
import torch

from helpers import BF16_REL
from oracle import ema_oracle as eo

pytestmark = pytest.mark.gpu


def _inputs(seed, b, L, h, d, dtype):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn((b, L, h, d), generator=g, device="cuda", dtype=torch.float32).to(dtype)
    a = torch.sigmoid(1.0 + 5.0 * torch.rand((b, L, h), generator=g, device="cuda"))
    w = 0.05 + 1.5 * torch.rand((b, L, h), generator=g, device="cuda")
    c = torch.randn((b, L, h), generator=g, device="cuda")
    return x, a, w, c


def _reference(x, a, w, c, init=None):
    """(y, s) in float64-accumulated fp32: the states s and the weighted output y."""
    xn = x.float().cpu().numpy()
    u = xn if w is None else xn * w.cpu().numpy()[..., None]
    A = np.log(a.cpu().numpy().astype(np.float64)).astype(np.float32)
    s = eo.fwd(np.ascontiguousarray(u, dtype=np.float32), A, convention=eo.REFERENCE, acc64=True)
    assert init is None
    y = s if c is None else s * c.cpu().numpy()[..., None]
    return y, s


def _check(got, ref, dtype, what):
    g = got.float().cpu().numpy()
    if dtype == torch.float32:
        assert np.abs(g - ref).max() <= 1e-4 * max(1.0, np.abs(ref).max()), what
    else:
        assert np.abs(g - ref).max() <= BF16_REL * np.abs(ref).max(), what


SHAPES = [
    (2, 300, 2, 64),
    (1, 1000, 3, 100),     # d not a multiple of 8: narrow vectors in the CUDA-core kernel, ragged channel tile otherwise
    (2, 129, 2, 24),
    (5, 300, 2, 1024),     # bf16: work items of two channel tiles
    (19, 300, 8, 256),     # bf16: 304 two-tile items, cut across thread blocks
]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("which", ["both", "in", "out"])
def test_weighted_forward_matches_oracle(shape, dtype, which, ema_lib):
    from ema_b200 import ops
    b, L, h, d = shape
    x, a, w, c = _inputs(300 + L + d, b, L, h, d, dtype)
    if which == "in":
        c = None
    if which == "out":
        w = None
    log_a = torch.log(a)
    r = ops.ema_fwd(x, log_a, prescaled_log=True, in_weight=w, out_weight=c, want_final=True, want_tile_states=True)
    torch.cuda.synchronize()
    if dtype == torch.bfloat16 and d % 8 == 0:
        assert ema_lib.ema_b200_last_path() == 1
    y_ref, s_ref = _reference(x, a, w, c)
    _check(r["y"], y_ref, dtype, "y")
    _check(r["final_state"], np.ascontiguousarray(s_ref[:, -1]), dtype, "final state (unweighted)")
    # saved states: the state entering every 128-step tile, unweighted
    nt = r["tile_states"].shape[1]
    ts = r["tile_states"].view(b, h, nt, d).float().cpu().numpy()
    for k in range(1, nt):
        ref_k = s_ref[:, 128 * k - 1]      # [b, h, d]
        err = np.abs(ts[:, :, k] - ref_k).max()
        assert err <= (1e-4 if dtype == torch.float32 else BF16_REL) * max(1.0, np.abs(s_ref).max()), f"tile state {k}"
    assert ema_lib.ema_b200_device_status(0) == 0


def test_input_weight_replaces_the_conventions_weight(ema_lib):
    """With the decay given as `a` (not its log) the input weight still replaces 1 - a; in_weight = 1 - a gives the
    plain EMA bit for bit in fp32."""
    from ema_b200 import ops
    x, a, _, _ = _inputs(11, 2, 520, 2, 128, torch.float32)
    plain = ops.ema_fwd(x, a)["y"]
    weighted = ops.ema_fwd(x, a, in_weight=(1.0 - a))["y"]
    assert torch.equal(plain, weighted)


def test_weights_need_a_per_step_decay(ema_lib):
    from ema_b200 import ops
    x, a, w, _ = _inputs(12, 1, 64, 2, 32, torch.float32)
    with pytest.raises(ValueError):
        ops.ema_fwd(x, a[0, 0].contiguous(), in_weight=w)
    with pytest.raises(ValueError):
        ops.ema_fwd(x, a, in_weight=w[:, :10])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_output_weight_alone_keeps_the_conventions_input_weight(dtype, ema_lib):
    """Without an input-weight tensor the input weight stays the convention's 1 - a: y = c * ema(x, a)."""
    from ema_b200 import ops
    x, a, _, c = _inputs(21, 3, 700, 2, 192, dtype)
    plain = ops.ema_fwd(x, a)["y"].float()
    got = ops.ema_fwd(x, a, out_weight=c)["y"].float()
    want = c.unsqueeze(-1) * plain
    if dtype == torch.float32:
        assert torch.equal(got, want)
    else:   # the plain result was rounded to bf16 before the multiplication, the weighted one after it
        assert float((got - want).abs().max()) <= BF16_REL * float(want.abs().max())


# ---- weighted backward ---------------------------------------------------------------------------------------------
def _loop_with_grads(x, dec, w, c, dy, log_conv, init, dfin):
    """The weighted recurrence as a float64 torch loop (the sequential definition of the reference's loops,
    kernels/tests/ema_bwd/_ema_full_bwd.py:24-34, with per-step input and output weights), differentiated by autograd."""
    leaves = {k: (None if v is None else v.detach().double().cpu().requires_grad_(True))
              for k, v in dict(x=x, dec=dec, w=w, c=c, init=init).items()}
    xx, dd = leaves["x"], leaves["dec"]
    b, L, h, d = xx.shape
    a = torch.exp(dd) if log_conv else dd
    win = leaves["w"] if w is not None else (torch.ones_like(a) if log_conv else 1.0 - a)
    s = torch.zeros(b, h, d, dtype=torch.float64) if init is None else leaves["init"]
    ys = []
    for t in range(L):
        s = a[:, t].unsqueeze(-1) * s + win[:, t].unsqueeze(-1) * xx[:, t]
        ys.append(s if c is None else leaves["c"][:, t].unsqueeze(-1) * s)
    y = torch.stack(ys, dim=1)
    loss = (y * dy.double().cpu()).sum()
    if dfin is not None:
        loss = loss + (s * dfin.double().cpu()).sum()
    loss.backward()
    return {k: (None if v is None else v.grad) for k, v in leaves.items()}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("which", ["both", "in", "out"])
@pytest.mark.parametrize("log_conv", [False, True])
@pytest.mark.parametrize("shape", [(2, 300, 2, 64), (1, 261, 3, 100), (3, 130, 2, 256)])
def test_weighted_backward_matches_autograd_of_the_loop(shape, log_conv, which, dtype, ema_lib):
    from ema_b200 import ops
    b, L, h, d = shape
    x, a, w, c = _inputs(40 + L, b, L, h, d, dtype)
    g = torch.Generator(device="cuda").manual_seed(7)
    dy = torch.randn((b, L, h, d), generator=g, device="cuda").to(dtype)
    init = torch.randn((b, h, d), generator=g, device="cuda")
    dfin = torch.randn((b, h, d), generator=g, device="cuda")
    dec = torch.log(a) if log_conv else a
    w_ = w if which in ("both", "in") else None
    c_ = c if which in ("both", "out") else None
    f = ops.ema_fwd(x, dec, prescaled_log=log_conv, init_state=init, want_tile_states=True, in_weight=w_, out_weight=c_)
    r = ops.ema_bwd_weighted(x, dec, dy, f["tile_states"], in_weight=w_, out_weight=c_, prescaled_log=log_conv,
                             dfinal_state=dfin, want_dinit=True)
    torch.cuda.synchronize()
    ref = _loop_with_grads(x.float(), dec, w_, c_, dy.float(), log_conv, init, dfin)

    def close(got, want, what):
        got, want = got.float().cpu(), want.float()
        scale = max(float(want.abs().max()), 1e-6)
        err = float((got - want).abs().max())
        tol = BF16_REL * scale if dtype == torch.bfloat16 else 1e-4 + 2e-5 * scale
        assert err <= tol, f"{what}: {err:.3e} > {tol:.3e} (scale {scale:.3e})"

    close(r["dx"], ref["x"], "dx")
    close(r["ddecay"], ref["dec"], "ddecay")
    close(r["dinit_state"], ref["init"], "dinit")
    if w_ is not None:
        close(r["din_weight"], ref["w"], "din_weight")
    else:
        assert "din_weight" not in r
    if c_ is not None:
        close(r["dout_weight"], ref["c"], "dout_weight")
    assert ema_lib.ema_b200_device_status(1) == 0


def test_weighted_backward_argument_checks(ema_lib):
    from ema_b200 import ops
    x, a, w, c = _inputs(3, 1, 64, 2, 32, torch.float32)
    ts = ops.ema_fwd(x, a, want_tile_states=True, in_weight=w)["tile_states"]
    with pytest.raises(ValueError):
        ops.ema_bwd_weighted(x, a[0, 0].contiguous(), x, ts, in_weight=w)          # per-head decay
    with pytest.raises(ValueError):
        ops.ema_bwd_weighted(x, a, x, ts, in_weight=w[:, :10])                     # weight of the wrong shape
    # no channels: every per-step gradient is an empty sum
    x0 = torch.zeros(1, 5, 2, 0, device="cuda")
    a0 = torch.full((1, 5, 2), 0.9, device="cuda")
    r = ops.ema_bwd_weighted(x0, a0, x0, torch.zeros(2, 1, 0, device="cuda"), in_weight=a0, out_weight=a0)
    assert bool((r["ddecay"] == 0).all()) and bool((r["din_weight"] == 0).all()) and bool((r["dout_weight"] == 0).all())
