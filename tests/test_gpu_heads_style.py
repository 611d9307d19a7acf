"""The heads-style entry point ema_chunk_scan_combined (drop-in for kernels/ema_combined.py:100 of the
reference) in the EMA special case, state size 1: against fixtures recorded from the reference's own entry point
(its Triton kernels under the CPU interpreter, tests/golden/heads_*.npz) and against the sequential fp64 loop of
oracle/ema_heads_loop.py, values and gradients."""
import os

import numpy as np
import pytest
import torch

from helpers import BF16_REL, FP32_ATOL
from oracle.ema_heads_loop import heads_loop, heads_loop_torch


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["heads_plain", "heads_full", "heads_seqidx"])
@pytest.mark.parametrize("grad", [False, True])
def test_heads_style_matches_the_reference_fixture(name, grad, ema_lib, golden_dir):
    """out and final_states equal what the reference's ema_chunk_scan_combined returned on the same inputs (A = -1:
    the reference ignores A, kernels/ema_chunk_state.py:95); both the fused inference route (no gradients) and the
    autograd route."""
    from kernels.ema_combined import ema_chunk_scan_combined
    g = np.load(os.path.join(golden_dir, name + ".npz"))
    assert int(g["meta_A_is_minus_one"][0]) == 1
    chunk, full = int(g["meta"][6]), bool(g["meta"][7])
    t = {k: torch.tensor(g[k]).cuda() for k in g.files if k not in ("out", "final_states", "meta", "meta_A_is_minus_one")}
    if grad:
        t["x"].requires_grad_(True)
    kw = dict(dt_softplus=True, dt_limit=(0.001, 2.0)) if full else {}
    with torch.enable_grad() if grad else torch.no_grad():
        out, fin = ema_chunk_scan_combined(t["x"], t["dt"], t["A"], t["B"], t["C"], chunk, D=t.get("D"), z=t.get("z"),
                                           dt_bias=t.get("dt_bias"), initial_states=t.get("initial_states"),
                                           seq_idx=t.get("seq_idx"), return_final_states=True, **kw)
    for got, ref, what in ((out, g["out"], "out"), (fin, g["final_states"], "final_states")):
        err = float(np.abs(got.detach().float().cpu().numpy() - ref).max())
        tol = FP32_ATOL + 2e-5 * float(np.abs(ref).max())
        assert err <= tol, f"{name} {what}: {err:.3e} > {tol:.3e}"
    assert ema_lib.ema_b200_device_status(1) == 0


def _loop(x, dt, A, B, C, D, z, dt_bias, init, softplus, limit, seq_idx=None):
    """The sequential fp64 definition (oracle/ema_heads_loop.py, pinned against fixtures recorded from the
    reference's own entry point), on torch leaves so that autograd gives the gradients."""
    return heads_loop_torch(x, dt, A, B, C, D=D, z=z, dt_bias=dt_bias, initial_states=init, dt_softplus=softplus,
                            dt_limit=limit, seq_idx=seq_idx)


def _make(seed, b, L, h, p, g, dtype, full):
    gen = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=gen)
    t = {"x": r(b, L, h, p), "dt": 0.3 * r(b, L, h) - 1.0 if full else torch.rand(b, L, h, generator=gen) * 0.2 + 0.01,
         "A": -torch.rand(h, generator=gen) - 0.5, "B": torch.rand(b, L, g, 1, generator=gen),
         "C": torch.ones(b, L, g, 1) if not full else 0.5 + torch.rand(b, L, g, 1, generator=gen)}
    if full:
        t.update(D=r(h, p), z=r(b, L, h, p), dt_bias=0.1 * r(h), init=r(b, h, p, 1))
    lowp = {"x", "z"}   # the tensors that carry the activation dtype
    return {k: (v.to(dtype).float() if k in lowp else v) for k, v in t.items()}


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("full", [False, True])
def test_heads_style_matches_sequential_loop(dtype, full, ema_lib):
    from kernels.ema_combined import ema_chunk_scan_combined
    b, L, h, p, g = 2, 200, 4, 32, 2
    t = _make(5, b, L, h, p, g, dtype, full)
    kw = dict(dt_softplus=True, dt_limit=(0.001, 2.0)) if full else {}
    # reference values and gradients in fp64 on the CPU
    leaves = {k: v.double().requires_grad_(True) for k, v in t.items()}
    y_ref, fin_ref = _loop(leaves["x"], leaves["dt"], leaves["A"], leaves["B"], leaves["C"], leaves.get("D"),
                           leaves.get("z"), leaves.get("dt_bias"), leaves.get("init"), full, kw.get("dt_limit", (0.0, float("inf"))))
    gen = torch.Generator().manual_seed(11)
    dy = torch.randn(y_ref.shape, generator=gen).to(dtype).float()
    dfin = torch.randn(fin_ref.shape, generator=gen)
    (y_ref * dy.double()).sum().add((fin_ref * dfin.double()).sum()).backward()
    # the library
    dev = {k: (v.to(dtype) if k in ("x", "z") else v).cuda().requires_grad_(True) for k, v in t.items()}
    out, fin = ema_chunk_scan_combined(dev["x"], dev["dt"], dev["A"], dev["B"], dev["C"], 64, D=dev.get("D"),
                                       z=dev.get("z"), dt_bias=dev.get("dt_bias"), initial_states=dev.get("init"),
                                       return_final_states=True, **kw)
    assert out.dtype == dtype and out.shape == (b, L, h, p) and fin.shape == (b, h, p, 1)
    ((out.float() * dy.cuda()).sum() + (fin * dfin.cuda()).sum()).backward()

    def close(got, ref, what):
        got, ref = got.detach().float().cpu(), ref.detach().float()
        scale = max(float(ref.abs().max()), 1e-6)
        err = float((got - ref).abs().max())
        tol = BF16_REL * scale if dtype == torch.bfloat16 else FP32_ATOL + 2e-5 * scale
        assert err <= tol, f"{what}: max err {err:.3e} > {tol:.3e} (scale {scale:.3e})"

    close(out, y_ref, "out")
    close(fin, fin_ref, "final_states")
    for k in t:
        close(dev[k].grad, leaves[k].grad, f"d{k}")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sequence_ids_restart_the_state(dtype, ema_lib):
    from kernels.ema_combined import ema_chunk_scan_combined
    b, L, h, p, g = 2, 300, 2, 64, 1
    t = _make(8, b, L, h, p, g, dtype, False)
    seq_idx = torch.zeros(b, L, dtype=torch.int32)
    seq_idx[0, 100:] = 1
    seq_idx[0, 128:] = 2          # a restart exactly on a tile boundary
    seq_idx[1, 257:] = 5
    leaves = {k: v.double().requires_grad_(True) for k, v in t.items()}
    y_ref, fin_ref = _loop(leaves["x"], leaves["dt"], leaves["A"], leaves["B"], leaves["C"], None, None, None, None,
                           False, (0.0, float("inf")), seq_idx=seq_idx)
    dy = torch.randn(y_ref.shape, generator=torch.Generator().manual_seed(3)).to(dtype).float()
    (y_ref * dy.double()).sum().backward()
    dev = {k: (v.to(dtype) if k == "x" else v).cuda().requires_grad_(True) for k, v in t.items()}
    out, fin = ema_chunk_scan_combined(dev["x"], dev["dt"], dev["A"], dev["B"], dev["C"], 64, seq_idx=seq_idx.cuda(),
                                       return_final_states=True)
    (out.float() * dy.cuda()).sum().backward()
    tol = BF16_REL if dtype == torch.bfloat16 else 1e-4
    for got, ref, what in ((out, y_ref, "out"), (fin, fin_ref, "final"), (dev["x"].grad, leaves["x"].grad, "dx"),
                           (dev["dt"].grad, leaves["dt"].grad, "ddt"), (dev["B"].grad, leaves["B"].grad, "dB")):
        got, ref = got.detach().float().cpu(), ref.detach().float()
        assert bool(torch.isfinite(got).all()), what
        assert float((got - ref).abs().max()) <= tol * max(float(ref.abs().max()), 1.0), what


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_inference_path_equals_training_path(dtype, ema_lib):
    """Without gradients the entry point takes a shorter elementwise route around the same scan."""
    from kernels.ema_combined import ema_chunk_scan_combined
    b, L, h, p, g = 2, 260, 4, 64, 2
    t = _make(13, b, L, h, p, g, dtype, False)
    dev = {k: (v.to(dtype) if k == "x" else v).cuda() for k, v in t.items()}
    init = torch.randn(b, h, p, 1, device="cuda")
    with torch.no_grad():
        out0, fin0 = ema_chunk_scan_combined(dev["x"], dev["dt"], dev["A"], dev["B"], dev["C"], 64, initial_states=init,
                                             return_final_states=True)
    xg = dev["x"].clone().requires_grad_(True)
    out1, fin1 = ema_chunk_scan_combined(xg, dev["dt"], dev["A"], dev["B"], dev["C"], 64, initial_states=init,
                                         return_final_states=True)
    tol = BF16_REL if dtype == torch.bfloat16 else 1e-5
    assert float((out0.float() - out1.float()).abs().max()) <= tol * max(float(out1.float().abs().max()), 1.0)
    assert float((fin0 - fin1).abs().max()) <= tol * max(float(fin1.abs().max()), 1.0)


def test_rejects_what_is_not_the_ema_case():
    from kernels.ema_combined import ema_chunk_scan_combined
    x, dt, A = torch.zeros(1, 8, 2, 4), torch.zeros(1, 8, 2), -torch.ones(2)
    B2 = torch.zeros(1, 8, 1, 2)
    with pytest.raises(NotImplementedError):
        ema_chunk_scan_combined(x, dt, A, B2, B2, 4)                       # state size 2
    B1 = torch.zeros(1, 8, 1, 1)
    with pytest.raises(NotImplementedError):   # packed sequences without a seq_idx that restarts the state between them
        ema_chunk_scan_combined(x, dt, A, B1, B1, 4, cu_seqlens=torch.tensor([0, 4, 8]), return_varlen_states=True)
    with pytest.raises(AssertionError):         # varlen states need batch 1, as in the reference
        ema_chunk_scan_combined(x.repeat(2, 1, 1, 1), dt.repeat(2, 1, 1), A, B1.repeat(2, 1, 1, 1), B1.repeat(2, 1, 1, 1), 4,
                                cu_seqlens=torch.tensor([0, 8]), return_varlen_states=True)
    with pytest.raises(AssertionError):
        ema_chunk_scan_combined(x, dt[:, :4], A, B1, B1, 4)               # dt of the wrong length


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["heads_varlen", "heads_varlen_full"])
@pytest.mark.parametrize("grad", [False, True])
def test_varlen_states_match_the_reference_fixture(name, grad, ema_lib, golden_dir):
    """out, final_states and the state at the end of every packed sequence equal what the reference's entry point
    returned with return_varlen_states=True (batch 1; kernels/ema_combined.py:56-62)."""
    from kernels.ema_combined import ema_chunk_scan_combined
    g = np.load(os.path.join(golden_dir, name + ".npz"))
    chunk, full = int(g["meta"][6]), bool(g["meta"][7])
    skip = ("out", "final_states", "varlen_states", "meta", "meta_A_is_minus_one")
    t = {k: torch.tensor(g[k]).cuda() for k in g.files if k not in skip}
    if grad:
        t["x"].requires_grad_(True)
    kw = dict(dt_softplus=True, dt_limit=(0.001, 2.0)) if full else {}
    with torch.enable_grad() if grad else torch.no_grad():
        out, fin, var = ema_chunk_scan_combined(
            t["x"], t["dt"], t["A"], t["B"], t["C"], chunk, D=t.get("D"), z=t.get("z"), dt_bias=t.get("dt_bias"),
            initial_states=t.get("initial_states"), seq_idx=t["seq_idx"], cu_seqlens=t["cu_seqlens"],
            return_final_states=True, return_varlen_states=True, **kw)
        out2, var2 = ema_chunk_scan_combined(
            t["x"], t["dt"], t["A"], t["B"], t["C"], chunk, D=t.get("D"), z=t.get("z"), dt_bias=t.get("dt_bias"),
            initial_states=t.get("initial_states"), seq_idx=t["seq_idx"], cu_seqlens=t["cu_seqlens"],
            return_varlen_states=True, **kw)
    assert torch.equal(out, out2) and torch.equal(var, var2)
    assert var.shape == g["varlen_states"].shape and var.dtype == torch.float32
    for got, ref, what in ((out, g["out"], "out"), (fin, g["final_states"], "final_states"),
                           (var, g["varlen_states"], "varlen_states")):
        err = float(np.abs(got.detach().float().cpu().numpy() - ref).max())
        tol = FP32_ATOL + 2e-5 * float(np.abs(ref).max())
        assert err <= tol, f"{name} {what}: {err:.3e} > {tol:.3e}"
    if grad:   # forward only, as in the reference
        with pytest.raises(AssertionError):
            out.sum().backward()
    assert ema_lib.ema_b200_device_status(1) == 0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("chunk", [64, 256])
def test_varlen_states_on_long_packed_sequences(dtype, chunk, ema_lib):
    """Sequences that end on a chunk boundary, one step long, longer than several chunks, and an initial state;
    against the sequential loop."""
    from kernels.ema_combined import ema_chunk_scan_combined
    L, h, p, g = 1500, 4, 128, 2
    cu = [0, 1, 64, 65, 256, 300, 1024, 1499, 1500]
    gen = torch.Generator().manual_seed(5)
    x = torch.randn(1, L, h, p, generator=gen).to(dtype)
    dt = torch.rand(1, L, h, generator=gen) * 0.2 + 0.01
    A = -torch.rand(h, generator=gen) - 0.5
    B = torch.rand(1, L, g, 1, generator=gen)
    C = 0.5 + torch.rand(1, L, g, 1, generator=gen)
    init = torch.randn(1, h, p, 1, generator=gen)
    sid = torch.zeros(1, L, dtype=torch.int32)
    for i in range(len(cu) - 1):
        sid[0, cu[i]:cu[i + 1]] = i
    cu_t = torch.tensor(cu, dtype=torch.int32)
    with torch.no_grad():
        out, fin, var = ema_chunk_scan_combined(x.cuda(), dt.cuda(), A.cuda(), B.cuda(), C.cuda(), chunk,
                                                initial_states=init.cuda(), seq_idx=sid.cuda(), cu_seqlens=cu_t.cuda(),
                                                return_final_states=True, return_varlen_states=True)
    ref_out, ref_fin, ref_var = heads_loop(x.float().numpy(), dt.numpy(), A.numpy(), B.numpy(), C.numpy(),
                                           initial_states=init.numpy(), seq_idx=sid.numpy(), cu_seqlens=cu, chunk_size=chunk)
    rel = BF16_REL if dtype == torch.bfloat16 else 2e-5
    for got, ref, what in ((out, ref_out, "out"), (fin, ref_fin, "final"), (var, ref_var, "varlen")):
        err = float(np.abs(got.float().cpu().numpy() - ref).max())
        assert err <= FP32_ATOL + rel * float(np.abs(ref).max()), f"{what}: {err:.3e}"
    assert ema_lib.ema_b200_device_status(1) == 0
