"""The reference's combined entry points (same names and signatures) against its recorded outputs
and against its sequential loop."""
import os

import numpy as np
import pytest
import torch
from einops import rearrange

from oracle import ema_oracle as eo

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _lib(ema_lib):
    assert torch.cuda.is_available()


def cu(v):
    return torch.tensor(v, device="cuda")


def err(got, ref):
    return float(np.abs(got.detach().float().cpu().numpy() - ref).max())


@pytest.mark.parametrize("name", ["stages_ragged", "stages_even"])
def test_combined_fwd_and_bwd_against_reference(golden_dir, name):
    from kernels.ema_kernels.ema_combined_fwd import _ema_matmul_scan_combined_fwd, ema_matmul_scan_combined
    from kernels.ema_kernels_bwd.ema_combined_bwd import _ema_chunk_scan_combined_bwd
    g = np.load(os.path.join(golden_dir, name + ".npz"))
    _, B, L, T, Q = (int(v) for v in g["meta"])
    A, X, dout = cu(g["A"]), cu(g["X"]), cu(g["dout"])
    out, cs, states, final = _ema_matmul_scan_combined_fwd(A, X, Q)
    assert out.shape == (B, L, T) and cs.shape == g["cs"].shape and states.shape == g["chunk_start_states"].shape
    assert err(out, g["out"]) <= 1e-4 and err(out, g["loop_out"]) <= 1e-4
    assert err(cs, g["cs"]) <= 1e-5
    assert err(states, g["chunk_start_states"]) <= 1e-4
    assert err(final, g["final"]) <= 1e-4
    dx, ddA, out2 = _ema_chunk_scan_combined_bwd(dout, X, A, Q, recompute_output=True)
    assert ddA.shape == g["comb_ddA"].shape
    assert err(dx, g["loop_dX"]) <= 1e-4 and err(dx, g["comb_dx"]) <= 1e-4
    assert err(out2, g["loop_out"]) <= 1e-4
    dA = rearrange(ddA, "b c s -> b (c s)")[:, :L]
    scale = float(np.abs(g["loop_dA"]).max())
    assert err(dA, g["loop_dA"]) <= 1e-4 + 2e-5 * scale
    assert err(ddA, g["comb_ddA"]) <= 1e-4 + 3e-5 * scale
    assert torch.all(rearrange(ddA, "b c s -> b (c s)")[:, L:] == 0)
    # autograd wiring of the public function (the reference's backward is a stub)
    A_, X_ = A.clone().requires_grad_(True), X.clone().requires_grad_(True)
    ema_matmul_scan_combined(A_, X_, Q).backward(dout)
    assert err(X_.grad, g["loop_dX"]) <= 1e-4
    assert err(A_.grad, g["loop_dA"]) <= 1e-4 + 2e-5 * scale


def test_prefix_entry_point_matches_pweighted_loop():
    """kernels/ema.py::ema_scan_combined(x[B,T,D], p[B,T,1]) - the reference's smoke script compares
    it with its sequential loop at B2, L512, D64 (main.py:133-144)."""
    from kernels.ema import ema_scan_combined
    B, T, D = 2, 512, 64
    rs = np.random.RandomState(0)
    x = rs.standard_normal((B, T, D)).astype(np.float32)
    p = rs.random_sample((B, T, 1)).astype(np.float32)
    a = (1.0 - p)[..., 0]
    ref = eo.fwd(x[:, :, None, :], a[:, :, None])[:, :, 0]
    z = ema_scan_combined(cu(x), cu(p))
    assert z.shape == (B, T, D) and err(z, ref) <= 1e-4
    with pytest.raises(AssertionError):
        ema_scan_combined(cu(x).transpose(1, 2), cu(p))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_prefix_entry_point_values_and_gradients(dtype):
    """The prefix entry point in both element types, with the gradients the reference's backward leaves out
    (kernels/ema.py:366-367 returns None): against the sequential p-weighted loop and autograd through it."""
    from kernels.ema import ema_scan_combined
    from oracle import ema_loop_port as lp
    B, T, D = 3, 700, 256
    g = torch.Generator().manual_seed(4)
    x = torch.randn((B, T, D), generator=g).to(dtype)
    p = torch.sigmoid(-4.0 + 3.0 * torch.rand((B, T, 1), generator=g))     # long memory: 1 - p up to 0.98
    dz = torch.randn((B, T, D), generator=g).to(dtype)
    xr = x.float().clone().requires_grad_(True)
    pr = p.clone().requires_grad_(True)
    z_ref = lp.ema_loop_pweighted(xr, pr)
    (z_ref * dz.float()).sum().backward()
    xd, pd = x.cuda().requires_grad_(True), p.cuda().requires_grad_(True)
    z = ema_scan_combined(xd, pd)
    assert z.dtype == dtype and z.shape == (B, T, D)
    z.backward(dz.cuda())

    def close(got, want, what):
        got, want = got.detach().float().cpu(), want.detach().float()
        scale = max(float(want.abs().max()), 1e-6)
        tol = 2e-2 * scale if dtype == torch.bfloat16 else 1e-4 + 2e-5 * scale
        assert float((got - want).abs().max()) <= tol, what

    close(z, z_ref, "z")
    close(xd.grad, xr.grad, "dx")
    close(pd.grad, pr.grad, "dp")


def test_reference_argument_contracts():
    from kernels.ema_kernels.ema_state_fwd import _ema_chunk_state_fwd
    from kernels.ema_kernels.ema_state_pass import _ema_state_passing_fwd
    from kernels.ema_kernels_bwd.ema_state_passing_bwd_dstates import _ema_state_passing_bwd
    S = torch.zeros(2, 3, 8, device="cuda")
    cl = torch.zeros(2, 3, device="cuda")
    with pytest.raises(NotImplementedError):
        _ema_state_passing_fwd(S, cl, initial_states=torch.zeros(2, 8, device="cuda"))
    with pytest.raises(AssertionError):
        _ema_state_passing_bwd(S, cl, S, dfinal_states=torch.zeros(2, 8, device="cuda"))
    with pytest.raises(AssertionError):
        _ema_state_passing_bwd(S, cl, S, has_initial_states=True)
    with pytest.raises(AssertionError):
        _ema_chunk_state_fwd(torch.zeros(2, 8, 6, device="cuda").transpose(1, 2), torch.zeros(2, 1, 6, device="cuda"))
