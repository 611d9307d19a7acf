"""The CPU oracle against fixtures produced by running the reference project's own code
(tests/golden/make_golden.py): its sequential PyTorch loops + autograd, and its Triton stage
kernels under Triton's interpreter.  No GPU needed."""
import os

import numpy as np
import pytest
import torch

from golden_inputs import gen_inputs
from oracle import ema_loop_port as lp
from oracle import ema_oracle as eo
from oracle import ema_stages_np as st


def _load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name + ".npz"))


def _northstar_inputs(g):
    seed, b, L, h, d, ph = (int(v) for v in g["meta"])
    lo, hi = g["lohi"]
    x, a, dy = gen_inputs(seed, b, L, h, d, lo, hi, bool(ph))
    assert np.array_equal(a, g["a"]), "seeded generator no longer reproduces the fixture inputs"
    return x, a, dy


@pytest.mark.parametrize("name", ["northstar_c1", "northstar_perhead", "northstar_ragged"])
@pytest.mark.parametrize("acc64", [False, True])
def test_c_oracle_matches_reference_loop_and_autograd(golden_dir, name, acc64):
    g = _load(golden_dir, name)
    x, a, dy = _northstar_inputs(g)
    y = eo.fwd(x, a, acc64=acc64)
    dx, da = eo.bwd(x, a, dy, acc64=acc64)
    if not acc64:
        # same fp32 operation order as the reference's p-weighted loop: bit exact
        assert np.array_equal(y, g["y"])
    assert np.abs(y - g["y"]).max() <= 1e-6
    assert np.abs(dx - g["dx"]).max() <= 2e-6
    assert np.abs(da - g["da"]).max() <= 3e-6 * np.abs(g["da"]).max()


@pytest.mark.parametrize("name", ["stages_ragged", "stages_even"])
def test_c_oracle_reference_convention(golden_dir, name):
    g = _load(golden_dir, name)
    A, X, dout = g["A"], g["X"], g["dout"]
    Q = int(g["meta"][4])
    y, states, final = eo.fwd(X[:, :, None, :], A[:, :, None], convention=eo.REFERENCE, chunk=Q)
    dx, dA = eo.bwd(X[:, :, None, :], A[:, :, None], dout[:, :, None, :], convention=eo.REFERENCE)
    assert np.abs(y[:, :, 0] - g["loop_out"]).max() <= 1e-5
    assert np.abs(dx[:, :, 0] - g["loop_dX"]).max() <= 1e-5
    assert np.abs(dA[:, :, 0] - g["loop_dA"]).max() <= 3e-6 * np.abs(g["loop_dA"]).max()
    # also equals what the reference's Triton pipeline produced
    assert np.abs(y[:, :, 0] - g["out"]).max() <= 1e-5
    assert np.abs(states[:, 0] - g["chunk_start_states"]).max() <= 1e-5
    assert np.abs(final[:, 0] - g["final"]).max() <= 1e-5


@pytest.mark.parametrize("name", ["stages_ragged", "stages_even"])
def test_numpy_stages_match_reference_triton_kernels(golden_dir, name):
    g = _load(golden_dir, name)
    A, X, dout = g["A"], g["X"], g["dout"]
    _, B, L, T, Q = (int(v) for v in g["meta"])
    e = lambda a, b: float(np.abs(a - b).max())
    assert e(st.chunk_cumsum(A, Q), g["cs"]) <= 5e-6
    assert e(st.chunk_state(X, g["cs"]), g["S"]) <= 2e-5
    h, fin = st.state_passing_fwd(g["S"], g["cs"][..., -1])
    assert e(h, g["chunk_start_states"]) <= 1e-5 and e(fin, g["final"]) <= 1e-5
    assert e(st.chunk_scan(X, g["cs"], g["chunk_start_states"]), g["out"]) <= 1e-5
    assert e(st.bwd_dstates(g["cs"], dout), g["dh_scan"]) <= 1e-5
    dS, dl = st.state_passing_bwd(g["chunk_start_states"], g["cs"][..., -1], g["dh_scan"])
    assert e(dS, g["dS"]) <= 1e-5 and e(dl, g["ddA_last"]) <= 1e-5
    assert e(st.bwd_dx(g["cs"], dout, g["dS"], L), g["dx"]) <= 1e-5
    assert e(st.bwd_db(X, g["cs"], g["dS"], raw=True), g["db_raw"]) <= 2e-5
    assert e(st.bwd_db(X, g["cs"], g["dS"]), g["db"]) <= 5e-5
    assert e(st.bwd_dc(g["chunk_start_states"], g["cs"], dout), g["dc"]) <= 2e-5
    assert e(st.bwd_dacs(X, g["cs"], dout), g["dacs"]) <= 1e-6 * max(1.0, np.abs(g["dacs"]).max()) * 300
    dx, ddA = st.combined_bwd(dout, X, A, Q)
    assert e(dx, g["comb_dx"]) <= 2e-5
    assert e(ddA, g["comb_ddA"]) <= 1e-6 * max(1.0, np.abs(g["comb_ddA"]).max()) * 300


def test_torch_loop_port_is_the_reference_loop(golden_dir):
    g = _load(golden_dir, "northstar_ragged")
    x, a, dy = _northstar_inputs(g)
    y, dx, da = lp.north_star_fwd_bwd(torch.tensor(x), torch.tensor(a), torch.tensor(dy))
    assert np.array_equal(y.numpy(), g["y"])
    assert np.abs(dx.numpy() - g["dx"]).max() <= 1e-6
    assert np.abs(da.numpy() - g["da"]).max() <= 1e-4


def test_two_conventions_agree():
    """y(a, x) in the north-star convention == y(log a, (1-a) x) in the reference convention."""
    x, a, dy = gen_inputs(5, 2, 100, 2, 8, 2.0, 6.0)
    y0 = eo.fwd(x, a, acc64=True)
    y1 = eo.fwd((1 - a)[..., None] * x, np.log(a), convention=eo.REFERENCE, acc64=True)
    assert np.abs(y0 - y1).max() <= 1e-6
    # chain rule between the two parametrisations: dx = (1-a) du, da = dA / a - sum_d du x
    dx0, da0 = eo.bwd(x, a, dy, acc64=True)
    du, dA = eo.bwd((1 - a)[..., None] * x, np.log(a), dy, convention=eo.REFERENCE, acc64=True)
    assert np.abs(dx0 - (1 - a)[..., None] * du).max() <= 1e-6
    assert np.abs(da0 - (dA / a - (du * x).sum(-1))).max() <= 1e-4 * np.abs(da0).max()


def test_edge_shapes():
    for (b, L, h, d) in [(1, 1, 1, 1), (2, 0, 2, 4), (1, 5, 3, 0)]:
        x, a, dy = gen_inputs(3, b, L, h, d, 2.0, 6.0)
        y = eo.fwd(x, a)
        dx, da = eo.bwd(x, a, dy)
        assert y.shape == x.shape and dx.shape == x.shape and da.shape == a.shape
    x, a, dy = gen_inputs(3, 1, 1, 1, 4, 2.0, 6.0)
    assert np.allclose(eo.fwd(x, a), (1 - a)[..., None] * x)


@pytest.mark.parametrize("name", ["heads_plain", "heads_full", "heads_seqidx"])
def test_heads_loop_matches_the_reference_entry_point(name, golden_dir):
    """oracle/ema_heads_loop.py (numpy, and its torch twin used for gradients) against out / final_states recorded
    from the reference's ema_chunk_scan_combined (kernels/ema_combined.py:100) under the Triton interpreter."""
    import torch
    from oracle.ema_heads_loop import heads_loop, heads_loop_torch
    g = np.load(os.path.join(golden_dir, name + ".npz"))
    full = bool(g["meta"][7])
    opt = lambda k: g[k] if k in g.files else None
    kw = dict(dt_softplus=True, dt_limit=(0.001, 2.0)) if full else {}
    out, fin = heads_loop(g["x"], g["dt"], g["A"], g["B"], g["C"], D=opt("D"), z=opt("z"), dt_bias=opt("dt_bias"),
                          initial_states=opt("initial_states"), seq_idx=opt("seq_idx"), **kw)
    scale = float(np.abs(g["out"]).max())
    assert np.abs(out - g["out"]).max() <= 1e-5 * max(scale, 1.0)
    assert np.abs(fin - g["final_states"]).max() <= 1e-5 * max(float(np.abs(g["final_states"]).max()), 1.0)
    tt = lambda k: None if opt(k) is None else torch.tensor(g[k]).double() if g[k].dtype != np.int32 else torch.tensor(g[k])
    out_t, fin_t = heads_loop_torch(tt("x"), tt("dt"), tt("A"), tt("B"), tt("C"), D=tt("D"), z=tt("z"),
                                    dt_bias=tt("dt_bias"), initial_states=tt("initial_states"), seq_idx=tt("seq_idx"), **kw)
    assert np.abs(out_t.numpy() - out).max() <= 1e-9 * max(scale, 1.0)
    assert np.abs(fin_t.numpy() - fin).max() <= 1e-9 * max(scale, 1.0)


@pytest.mark.parametrize("name", ["heads_varlen", "heads_varlen_full"])
def test_heads_loop_varlen_states_match_the_reference(name, golden_dir):
    """The state at the end of every packed sequence (return_varlen_states, kernels/ema_combined.py:56-62 and
    kernels/ema_chunk_state.py:578 of the reference), recorded from the reference's entry point with batch 1 and a
    seq_idx that marks the same boundaries as cu_seqlens."""
    from oracle.ema_heads_loop import heads_loop
    g = np.load(os.path.join(golden_dir, name + ".npz"))
    full = bool(g["meta"][7])
    opt = lambda k: g[k] if k in g.files else None
    kw = dict(dt_softplus=True, dt_limit=(0.001, 2.0)) if full else {}
    out, fin, varlen = heads_loop(g["x"], g["dt"], g["A"], g["B"], g["C"], D=opt("D"), z=opt("z"), dt_bias=opt("dt_bias"),
                                  initial_states=opt("initial_states"), seq_idx=g["seq_idx"], cu_seqlens=g["cu_seqlens"],
                                  chunk_size=int(g["meta"][6]), **kw)
    for got, ref in ((out, g["out"]), (fin, g["final_states"]), (varlen, g["varlen_states"])):
        assert got.shape == ref.shape
        assert np.abs(got - ref).max() <= 1e-5 * max(float(np.abs(ref).max()), 1.0)
