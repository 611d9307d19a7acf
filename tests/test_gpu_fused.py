"""Fused forward/backward through the C ABI (via the ctypes host code) against the CPU oracle."""
import os

import numpy as np
import pytest
import torch

from golden_inputs import gen_inputs
from helpers import assert_close_fp32, check_outputs, make_inputs, oracle_fwd_bwd
from oracle import ema_oracle as eo

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _lib(ema_lib):
    assert torch.cuda.is_available()
    return ema_lib


def _ema():
    import ema_b200
    return ema_b200


SHAPES = [
    # b, L, h, d
    (2, 256, 2, 64),     # the CPU-oracle configuration
    (1, 1, 1, 8),
    (1, 63, 1, 8),
    (1, 64, 2, 16),
    (2, 65, 1, 24),      # d not a multiple of the channel tile
    (1, 200, 3, 100),
    (2, 131, 2, 7),      # odd d: scalar path
    (1, 1000, 1, 512),
    (1, 777, 2, 1024),
]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("per_head", [False, True])
def test_fwd_bwd_matches_oracle(shape, dtype, per_head):
    b, L, h, d = shape
    x, a, dy, np_in = make_inputs(100 + L + d, b, L, h, d, per_head=per_head, dtype=dtype)
    y_ref, dx_ref, da_ref = oracle_fwd_bwd(np_in)
    x.requires_grad_(True)
    a.requires_grad_(True)
    y = _ema().ema(x, a)
    y.backward(dy)
    check_outputs(dtype, y, y_ref, "y")
    check_outputs(dtype, x.grad, dx_ref, "dx")
    check_outputs(dtype, a.grad, da_ref, "da", grad_of_decay=True)
    assert y.dtype == dtype and x.grad.dtype == dtype and a.grad.dtype == torch.float32


@pytest.mark.parametrize("name", ["northstar_c1", "northstar_perhead", "northstar_ragged"])
def test_reference_goldens(golden_dir, name):
    """Against y/dx/da recorded from the reference's own sequential loop and autograd."""
    g = np.load(os.path.join(golden_dir, name + ".npz"))
    seed, b, L, h, d, ph = (int(v) for v in g["meta"])
    x, a, dy = gen_inputs(seed, b, L, h, d, *g["lohi"], bool(ph))
    xt = torch.tensor(x, device="cuda", requires_grad=True)
    at = torch.tensor(a, device="cuda", requires_grad=True)
    y = _ema().ema(xt, at)
    y.backward(torch.tensor(dy, device="cuda"))
    assert_close_fp32(y, g["y"], "y")
    assert_close_fp32(xt.grad, g["dx"], "dx")
    assert_close_fp32(at.grad, g["da"], "da", scale_rel=2e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_long_memory_decay(dtype):
    """sigmoid(U(3,8)) decays: carries across many tiles matter."""
    b, L, h, d = 1, 4096, 2, 64
    x, a, dy, np_in = make_inputs(7, b, L, h, d, lo=3.0, hi=8.0, dtype=dtype)
    y_ref, dx_ref, da_ref = oracle_fwd_bwd(np_in)
    x.requires_grad_(True)
    a.requires_grad_(True)
    y = _ema().ema(x, a)
    y.backward(dy)
    check_outputs(dtype, y, y_ref, "y")
    check_outputs(dtype, x.grad, dx_ref, "dx")
    check_outputs(dtype, a.grad, da_ref, "da", grad_of_decay=True)


def test_strided_view_equals_contiguous():
    """x given as a [b,L,h,d] view of a larger buffer (no physical transpose) gives the same bits."""
    E = _ema()
    b, L, h, d = 2, 150, 3, 32
    big = torch.randn(b, L, h, 2 * d, device="cuda")
    xv = big[..., :d]
    a = torch.sigmoid(2 + 4 * torch.rand(b, L, h, device="cuda"))
    y1 = E.ema_fwd(xv, a)["y"]
    y2 = E.ema_fwd(xv.contiguous(), a)["y"]
    assert torch.equal(y1, y2)
    # heads folded differently: [b,h,L,d] storage viewed as [b,L,h,d]
    xs = torch.randn(b, h, L, d, device="cuda").permute(0, 2, 1, 3)
    a_s = torch.sigmoid(2 + 4 * torch.rand(b, h, L, device="cuda")).permute(0, 2, 1)
    y3 = E.ema_fwd(xs, a_s)["y"]
    y4 = E.ema_fwd(xs.contiguous(), a_s.contiguous())["y"]
    assert torch.equal(y3, y4)


def test_prescaled_log_convention_and_chunk_states():
    """The reference's (A_ema, X_ema) convention, its chunk-start states and final state."""
    E = _ema()
    b, L, h, d, Q = 2, 300, 2, 40, 64
    rs = np.random.RandomState(3)
    A = (-0.2 * rs.random_sample((b, L, h))).astype(np.float32)
    U = rs.standard_normal((b, L, h, d)).astype(np.float32)
    dy = rs.standard_normal((b, L, h, d)).astype(np.float32)
    y_ref, st_ref, fin_ref = eo.fwd(U, A, convention=eo.REFERENCE, chunk=Q, acc64=True)
    du_ref, dA_ref = eo.bwd(U, A, dy, convention=eo.REFERENCE, acc64=True)
    Ut, At, gt = (torch.tensor(v, device="cuda") for v in (U, A, dy))
    r = E.ema_fwd(Ut, At, chunk=Q, prescaled_log=True, want_chunk_states=True, want_tile_states=True,
                  want_final=True, want_log_decay_sum=True)
    assert_close_fp32(r["y"], y_ref, "y")
    assert_close_fp32(r["chunk_states"], st_ref, "chunk states")
    assert_close_fp32(r["final_state"], fin_ref, "final state")
    assert_close_fp32(r["log_decay_sum"], A.sum(1), "log decay sum", scale_rel=2e-5)
    g = E.ema_bwd(Ut, At, gt, r["tile_states"], prescaled_log=True)
    assert_close_fp32(g["dx"], du_ref, "du")
    assert_close_fp32(g["ddecay"], dA_ref, "dA", scale_rel=2e-5)


@pytest.mark.parametrize("Q", [1, 7, 64, 100, 512])
def test_chunk_states_any_chunk_size(Q):
    E = _ema()
    b, L, h, d = 1, 260, 2, 16
    x, a, _, np_in = make_inputs(11, b, L, h, d)
    _, st_ref, fin_ref = eo.fwd(np_in[0], np_in[1], chunk=Q, acc64=True)
    r = E.ema_fwd(x, a, chunk=Q, want_chunk_states=True, want_final=True)
    assert_close_fp32(r["chunk_states"], st_ref, "chunk states")
    assert_close_fp32(r["final_state"], fin_ref, "final")


def test_init_and_final_state_split_equals_whole():
    """Scanning [0,L1) then [L1,L) with the carried state equals scanning [0,L) - forward and backward."""
    E = _ema()
    b, L, h, d, L1 = 2, 333, 2, 48, 140
    x, a, dy, np_in = make_inputs(21, b, L, h, d)
    whole = E.ema_fwd(x, a, want_tile_states=True)
    gw = E.ema_bwd(x, a, dy, whole["tile_states"])
    f1 = E.ema_fwd(x[:, :L1], a[:, :L1], want_final=True, want_tile_states=True)
    f2 = E.ema_fwd(x[:, L1:], a[:, L1:], init_state=f1["final_state"], want_tile_states=True)
    assert_close_fp32(torch.cat([f1["y"], f2["y"]], 1), whole["y"].cpu().numpy(), "split forward")
    g2 = E.ema_bwd(x[:, L1:], a[:, L1:], dy[:, L1:], f2["tile_states"], want_dinit=True)
    g1 = E.ema_bwd(x[:, :L1], a[:, :L1], dy[:, :L1], f1["tile_states"], dfinal_state=g2["dinit_state"])
    assert_close_fp32(torch.cat([g1["dx"], g2["dx"]], 1), gw["dx"].cpu().numpy(), "split dx")
    assert_close_fp32(torch.cat([g1["ddecay"], g2["ddecay"]], 1), gw["ddecay"].cpu().numpy(), "split da", scale_rel=2e-5)


def test_stop_below_rescans_only_the_prefix():
    """With a carry that dies out, a prefix re-scan (stop_below) reproduces the full result."""
    E = _ema()
    b, L, h, d = 1, 2048, 2, 32
    x, a, _, _ = make_inputs(31, b, L, h, d, lo=0.0, hi=2.0)   # a in 0.5..0.88: short memory
    init = torch.randn(b, h, d, device="cuda")
    full = E.ema_fwd(x, a, init_state=init, want_tile_states=True)
    zero = E.ema_fwd(x, a, want_tile_states=True)
    fixed = E.ema_fwd(x, a, init_state=init, stop_below=1e-12, out=zero["y"], tile_states=zero["tile_states"])
    assert torch.allclose(fixed["y"], full["y"], atol=1e-6, rtol=0)
    assert torch.allclose(fixed["tile_states"], full["tile_states"], atol=1e-6, rtol=0)
    # and it really stopped early: the tail of a poisoned output buffer is untouched
    poison = torch.full_like(full["y"], 7.0)
    E.ema_fwd(x, a, init_state=init, stop_below=1e-12, out=poison)
    assert torch.all(poison[:, -64:] == 7.0) and not torch.any(poison[:, :64] == 7.0)


def test_bitwise_deterministic():
    E = _ema()
    x, a, dy, _ = make_inputs(41, 2, 700, 2, 256, dtype=torch.bfloat16)
    outs = []
    for _ in range(2):
        f = E.ema_fwd(x, a, want_tile_states=True)
        g = E.ema_bwd(x, a, dy, f["tile_states"])
        outs.append((f["y"].clone(), g["dx"].clone(), g["ddecay"].clone()))
    for u, v in zip(*outs):
        assert torch.equal(u, v)


def test_empty_and_bad_arguments():
    E = _ema()
    y = E.ema_fwd(torch.zeros(2, 0, 2, 8, device="cuda"), torch.zeros(2, 0, 2, device="cuda"), want_final=True)
    assert y["y"].shape == (2, 0, 2, 8) and torch.all(y["final_state"] == 0)
    # no channels: the decay gradient is an empty sum for every step (a caller's buffer must not keep its old contents)
    for dtype in (torch.float32, torch.bfloat16):
        x0 = torch.zeros(2, 5, 2, 0, device="cuda", dtype=dtype)
        a0 = torch.full((2, 5, 2), 0.9, device="cuda")
        ts0 = E.ema_fwd(x0, a0, want_tile_states=True)["tile_states"]
        r0 = E.ema_bwd(x0, a0, x0, ts0, ddecay=torch.full_like(a0, float("nan")))
        assert r0["dx"].shape == (2, 5, 2, 0) and bool((r0["ddecay"] == 0).all())
    with pytest.raises(ValueError):
        E.ema_fwd(torch.zeros(2, 4, 2, 8, device="cuda"), torch.zeros(2, 4, 3, device="cuda"))
    with pytest.raises(TypeError):
        E.ema_fwd(torch.zeros(2, 4, 2, 8, device="cuda", dtype=torch.float16), torch.zeros(2, device="cuda"))
    with pytest.raises(RuntimeError):
        E.ema_fwd(torch.zeros(2, 4, 2, 8), torch.zeros(2))
