"""Every stage kernel against the numpy restatement of the reference stage and against the outputs
recorded from the reference's Triton kernels (tests/golden/stages_*.npz)."""
import os

import numpy as np
import pytest
import torch

from oracle import ema_stages_np as st

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _lib(ema_lib):
    assert torch.cuda.is_available()


def cu(v, dtype=None):
    t = torch.tensor(v, device="cuda")
    return t.to(dtype) if dtype is not None else t


def err(got, ref):
    return float(np.abs(got.detach().float().cpu().numpy() - ref).max())


@pytest.mark.parametrize("name", ["stages_ragged", "stages_even"])
def test_stages_against_reference_goldens(golden_dir, name):
    from kernels.ema_kernels.ema_cumsum import ema_chunk_cumsum_fwd
    from kernels.ema_kernels.ema_scan_fwd import _ema_scan_fwd
    from kernels.ema_kernels.ema_state_fwd import _ema_chunk_state_fwd
    from kernels.ema_kernels.ema_state_pass import _ema_state_passing_fwd
    from kernels.ema_kernels_bwd.ema_chunk_scan_bwd_dc import _ema_chunk_scan_bwd_dC
    from kernels.ema_kernels_bwd.ema_chunk_scan_chunk_state_bwd_dx import _chunk_scan_chunk_state_bwd_dx
    from kernels.ema_kernels_bwd.ema_chunk_state_bwd_db import _ema_chunk_state_bwd_db
    from kernels.ema_kernels_bwd.ema_scan_bwd import _ema_chunk_scan_bwd_dstates
    from kernels.ema_kernels_bwd.ema_scan_da import _ema_chunk_scan_bwd_ddAcs_stable
    from kernels.ema_kernels_bwd.ema_state_passing_bwd_dstates import _ema_state_passing_bwd

    g = np.load(os.path.join(golden_dir, name + ".npz"))
    _, B, L, T, Q = (int(v) for v in g["meta"])
    A, X, dout = cu(g["A"]), cu(g["X"]), cu(g["dout"])
    cs = ema_chunk_cumsum_fwd(A, Q)
    assert cs.shape == g["cs"].shape and cs.dtype == torch.float32
    assert err(cs, g["cs"]) <= 1e-5
    cs_g = cu(g["cs"])
    assert err(_ema_chunk_state_fwd(X, cs_g), g["S"]) <= 1e-4
    h, fin = _ema_state_passing_fwd(cu(g["S"]), cs_g[..., -1], out_dtype=torch.float32)
    assert err(h, g["chunk_start_states"]) <= 1e-4 and err(fin, g["final"]) <= 1e-4
    h_g = cu(g["chunk_start_states"])
    assert err(_ema_scan_fwd(X, cs_g, h_g), g["out"]) <= 1e-4
    assert err(_ema_chunk_scan_bwd_dstates(cs_g, dout, dtype=torch.float32), g["dh_scan"]) <= 1e-4
    dS, ddA_last, none = _ema_state_passing_bwd(h_g, cs_g[..., -1], cu(g["dh_scan"]), chunk_size=Q)
    assert none is None
    assert err(dS, g["dS"]) <= 1e-4 and err(ddA_last, g["ddA_last"]) <= 1e-4
    dS_g = cu(g["dS"])
    assert err(_chunk_scan_chunk_state_bwd_dx(X, cs_g, dout, dS_g), g["dx"]) <= 1e-4
    assert err(_ema_chunk_state_bwd_db(X, cs_g, dS_g, raw_scale_gradient=True), g["db_raw"]) <= 1e-4
    assert err(_ema_chunk_state_bwd_db(X, cs_g, dS_g), g["db"]) <= 2e-4
    assert err(_ema_chunk_scan_bwd_dC(h_g, cs_g, dout), g["dc"]) <= 1e-4
    scale = max(1.0, float(np.abs(g["dacs"]).max()))
    assert err(_ema_chunk_scan_bwd_ddAcs_stable(X, cs_g, dout), g["dacs"]) <= 1e-4 + 2e-5 * scale


@pytest.mark.parametrize("B,L,T,Q", [(2, 300, 40, 64), (1, 1000, 128, 128), (3, 517, 16, 32), (1, 600, 200, 256)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_stages_against_numpy_restatement(B, L, T, Q, dtype):
    from ema_b200 import stages
    rs = np.random.RandomState(B * 1000 + L)
    A = (-0.05 * rs.random_sample((B, L))).astype(np.float32)
    X = cu(rs.standard_normal((B, L, T)).astype(np.float32), dtype)
    dout = cu(rs.standard_normal((B, L, T)).astype(np.float32), dtype)
    Xn, dn = X.float().cpu().numpy(), dout.float().cpu().numpy()
    tol = 1e-4 if dtype == torch.float32 else None

    def ok(got, ref, what, relscale=2e-5):
        e = err(got, ref)
        s = float(np.abs(ref).max())
        bound = (1e-4 + relscale * s) if tol else 2e-2 * max(s, 1e-6)
        assert e <= bound, f"{what}: {e:.3e} > {bound:.3e}"

    cs_n = st.chunk_cumsum(A, Q)
    cs = stages.chunk_cumsum(cu(A), Q)
    ok(cs, cs_n, "cs")
    S_n = st.chunk_state(Xn, cs_n)
    ok(stages.chunk_state(X, cs), S_n, "S")
    h_n, fin_n = st.state_passing_fwd(S_n, cs_n[..., -1])
    h, fin = stages.state_passing_fwd(cu(S_n), cs[..., -1])
    ok(h, h_n, "h"); ok(fin, fin_n, "final")
    ok(stages.chunk_scan(X, cs, cu(h_n)), st.chunk_scan(Xn, cs_n, h_n), "scan")
    dh_n = st.bwd_dstates(cs_n, dn)
    ok(stages.bwd_dstates(cs, dout), dh_n, "dstates")
    dS_n, dl_n = st.state_passing_bwd(h_n, cs_n[..., -1], dh_n)
    dS, dl = stages.state_passing_bwd(cu(h_n), cs[..., -1], cu(dh_n))
    ok(dS, dS_n, "dS"); ok(dl, dl_n, "ddA_last")
    ok(stages.bwd_dx(X, cs, dout, cu(dS_n)), st.bwd_dx(cs_n, dn, dS_n, L), "dx")
    ok(stages.bwd_db(X, cs, cu(dS_n), raw=True), st.bwd_db(Xn, cs_n, dS_n, raw=True), "db raw")
    ok(stages.bwd_db(X, cs, cu(dS_n)), st.bwd_db(Xn, cs_n, dS_n), "db")
    ok(stages.bwd_dc(cu(h_n), cs, dout), st.bwd_dc(h_n, cs_n, dn), "dc")
    ok(stages.bwd_dacs(X, cs, dout), st.bwd_dacs(Xn, cs_n, dn), "dacs")
