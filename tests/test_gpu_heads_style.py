"""The heads-style entry point ema_chunk_scan_combined (drop-in for kernels/ema_combined.py:100 of the
reference) in the EMA special case, state size 1: against a sequential fp64 loop, values and gradients."""
import pytest
import torch
import torch.nn.functional as F

from helpers import BF16_REL, FP32_ATOL


def _loop(x, dt, A, B, C, D, z, dt_bias, init, softplus, limit, seq_idx=None):
    """fp64 sequential definition (the recurrence of the reference's chunked kernels, ema_combined.py:12-66)."""
    b, L, h, p = x.shape
    rep = h // B.shape[2]
    d = dt if dt_bias is None else dt + dt_bias
    if softplus:
        d = torch.where(d <= 20.0, F.softplus(d), d)
    d = torch.clamp(d, min=limit[0], max=limit[1])
    Bh = B[..., 0].repeat_interleave(rep, dim=2)
    Ch = C[..., 0].repeat_interleave(rep, dim=2)
    s = torch.zeros((b, h, p), dtype=x.dtype) if init is None else init[..., 0]
    ys = []
    for t in range(L):
        if seq_idx is not None and t > 0:   # a new sequence starts from a zero state
            s = s * (seq_idx[:, t] == seq_idx[:, t - 1]).to(s.dtype).view(b, 1, 1)
        s = torch.exp(d[:, t] * A).unsqueeze(-1) * s + (d[:, t] * Bh[:, t]).unsqueeze(-1) * x[:, t]
        ys.append(Ch[:, t].unsqueeze(-1) * s)
    y = torch.stack(ys, dim=1)
    if D is not None:
        y = y + x * (D.unsqueeze(-1) if D.dim() == 1 else D)
    if z is not None:
        y = y * F.silu(z)
    return y, s.unsqueeze(-1)


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
    with pytest.raises(NotImplementedError):
        ema_chunk_scan_combined(x, dt, A, B1, B1, 4, cu_seqlens=torch.tensor([0, 8]), return_varlen_states=True)
    with pytest.raises(AssertionError):
        ema_chunk_scan_combined(x, dt[:, :4], A, B1, B1, 4)               # dt of the wrong length
