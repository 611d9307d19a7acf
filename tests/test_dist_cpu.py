"""The multi-GPU host logic on CPU ranks (gloo, world_size 2 and 4): the carry exchange of the
sequence-parallel mode and the gradient all-reduce of the row-sharded mode.  The CUDA scan is
replaced by a small numpy stand-in with the same call interface, so what is tested is the exchange
algebra (fold order, log-domain decay products, prefix / suffix re-scan), not the kernels."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ema_b200 import dist as ema_dist
from golden_inputs import gen_inputs
from oracle import ema_oracle as eo


class NumpyScan:
    """Stand-in for ema_b200.ops on CPU tensors: plain sequential loops, float64."""

    @staticmethod
    def _a_full(x, a):
        b, L, h, d = x.shape
        an = a.detach().numpy().astype(np.float64)
        return np.broadcast_to(an.reshape(1, 1, h), (b, L, h)) if an.ndim == 1 else an

    @classmethod
    def ema_fwd(cls, x, a, *, want_tile_states=False, want_final=False, want_log_decay_sum=False, init_state=None,
                stop_below=0.0, out=None, tile_states=None, **_):
        xn = x.detach().numpy().astype(np.float64)
        af = cls._a_full(x, a)
        b, L, h, d = xn.shape
        z = np.zeros((b, h, d)) if init_state is None else init_state.numpy().astype(np.float64)
        y = np.empty_like(xn)
        start = z.copy()
        run = np.ones((b, h))
        stop_at = L
        for t in range(L):
            z = af[:, t, :, None] * z + (1 - af[:, t, :, None]) * xn[:, t]
            y[:, t] = z
            run = run * af[:, t]
            if stop_below > 0 and (t + 1) % 8 == 0 and run.max() < stop_below:
                stop_at = t + 1
                break
        res = {}
        if out is not None:
            out[:, :stop_at] = torch.tensor(y[:, :stop_at], dtype=out.dtype)
            res["y"] = out
        else:
            res["y"] = torch.tensor(y, dtype=x.dtype)
        # the stand-in's "saved states" are just the state entering the segment
        ts = tile_states if tile_states is not None else torch.zeros(b, h, d, dtype=torch.float64)
        ts.copy_(torch.tensor(start))
        res["tile_states"] = ts
        res["final_state"] = torch.tensor(z, dtype=torch.float32)
        res["log_decay_sum"] = torch.tensor(np.log(af).sum(1), dtype=torch.float32)
        return res

    @classmethod
    def ema_bwd(cls, x, a, dy, tile_states, *, want_dinit=False, dfinal_state=None, stop_below=0.0, dx=None,
                workspace=None, ddecay=None, **_):
        xn = x.detach().numpy().astype(np.float64)
        gn = dy.detach().numpy().astype(np.float64)
        af = cls._a_full(x, a)
        b, L, h, d = xn.shape
        z = tile_states.numpy().astype(np.float64)
        yprev = np.empty_like(xn)
        for t in range(L):
            yprev[:, t] = z
            z = af[:, t, :, None] * z + (1 - af[:, t, :, None]) * xn[:, t]
        lam = np.zeros((b, h, d)) if dfinal_state is None else dfinal_state.numpy().astype(np.float64)
        dxn = np.empty_like(xn)
        dan = np.zeros((b, L, h))
        a_next = np.ones((b, h))
        first = True
        for t in range(L - 1, -1, -1):
            lam = gn[:, t] + (lam if first else a_next[..., None] * lam)
            first = False
            dxn[:, t] = (1 - af[:, t, :, None]) * lam
            dan[:, t] = (lam * (yprev[:, t] - xn[:, t])).sum(-1)
            a_next = af[:, t]
        res = {"dx": torch.tensor(dxn, dtype=x.dtype), "workspace": torch.zeros(1)}
        res["ddecay"] = torch.tensor(dan.sum((0, 1)) if a.dim() == 1 else dan, dtype=torch.float32)
        res["dinit_state"] = torch.tensor(af[:, 0, :, None] * lam, dtype=torch.float32)
        return res


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, mode, per_head, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        b, L, h, d = 2, 64, 2, 8
        x, a, dy = gen_inputs(17, b, L, h, d, 0.0, 4.0, per_head)
        xt, at, gt = torch.tensor(x), torch.tensor(a), torch.tensor(dy)
        if mode == "sp":
            seg = L // world
            sl = slice(rank * seg, (rank + 1) * seg)
            xs = xt[:, sl].clone().requires_grad_(True)
            a_s = (at if per_head else at[:, sl]).clone().requires_grad_(True)
            y = ema_dist.ema_sequence_parallel(xs, a_s, backend=NumpyScan, stop_below=0.0)
            y.backward(gt[:, sl])
            q.put((rank, y.detach().numpy(), xs.grad.numpy(), a_s.grad.numpy()))
        else:
            xs, a_s = ema_dist.shard_rows(xt, at, rank, world)
            xs = xs.clone().requires_grad_(True)
            a_s = a_s.clone().requires_grad_(True)
            y = ema_dist.ema_row_sharded(xs, a_s, backend=NumpyScan, heads_replicated=True)
            b0, b1, h0, h1 = ema_dist.plan_row_shards(b, h, world)[rank]
            y.backward(gt[b0:b1, :, h0:h1])
            q.put((rank, y.detach().numpy(), xs.grad.numpy(), a_s.grad.numpy()))
    finally:
        dist.destroy_process_group()


def _run(world, mode, per_head):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, mode, per_head, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = {}
    for _ in range(world):
        r, y, dx, da = q.get(timeout=120)
        out[r] = (y, dx, da)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    return out


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("per_head", [False, True])
def test_sequence_parallel_equals_single_device(world, per_head):
    b, L, h, d = 2, 64, 2, 8
    x, a, dy = gen_inputs(17, b, L, h, d, 0.0, 4.0, per_head)
    y_ref = eo.fwd(x, a, acc64=True)
    dx_ref, da_ref = eo.bwd(x, a, dy, acc64=True)
    out = _run(world, "sp", per_head)
    y = np.concatenate([out[r][0] for r in range(world)], axis=1)
    dx = np.concatenate([out[r][1] for r in range(world)], axis=1)
    assert np.abs(y - y_ref).max() <= 1e-5
    assert np.abs(dx - dx_ref).max() <= 1e-5
    if per_head:
        for r in range(world):   # all-reduced: every rank holds the full gradient
            assert np.abs(out[r][2] - da_ref).max() <= 1e-4 * np.abs(da_ref).max()
    else:
        da = np.concatenate([out[r][2] for r in range(world)], axis=1)
        assert np.abs(da - da_ref).max() <= 1e-4 * np.abs(da_ref).max()


@pytest.mark.parametrize("per_head", [False, True])
def test_row_sharded_equals_single_device(per_head):
    world = 2
    b, L, h, d = 2, 64, 2, 8
    x, a, dy = gen_inputs(17, b, L, h, d, 0.0, 4.0, per_head)
    y_ref = eo.fwd(x, a, acc64=True)
    dx_ref, da_ref = eo.bwd(x, a, dy, acc64=True)
    out = _run(world, "rows", per_head)
    y = np.concatenate([out[r][0] for r in range(world)], axis=0)
    dx = np.concatenate([out[r][1] for r in range(world)], axis=0)
    assert np.abs(y - y_ref).max() <= 1e-5 and np.abs(dx - dx_ref).max() <= 1e-5
    if per_head:
        for r in range(world):
            assert np.abs(out[r][2] - da_ref).max() <= 1e-4 * np.abs(da_ref).max()
    else:
        da = np.concatenate([out[r][2] for r in range(world)], axis=0)
        assert np.abs(da - da_ref).max() <= 1e-4 * np.abs(da_ref).max()


def test_fold_helpers_match_direct_products():
    rs = np.random.RandomState(0)
    W, b, h, d = 5, 2, 3, 4
    finals = [torch.tensor(rs.standard_normal((b, h, d)), dtype=torch.float32) for _ in range(W)]
    logs = [torch.tensor(-rs.random_sample((b, h)), dtype=torch.float32) for _ in range(W)]
    for g in range(W):
        want = torch.zeros(b, h, d)
        for j in range(g):
            w = torch.exp(sum(logs[k] for k in range(j + 1, g)) if j + 1 < g else torch.zeros(b, h))
            want = want + w.unsqueeze(-1) * finals[j]
        assert torch.allclose(ema_dist.fold_carries(finals, logs, g), want, atol=1e-5)
        want = torch.zeros(b, h, d)
        for j in range(g + 1, W):
            w = torch.exp(sum(logs[k] for k in range(g + 1, j)) if g + 1 < j else torch.zeros(b, h))
            want = want + w.unsqueeze(-1) * finals[j]
        assert torch.allclose(ema_dist.fold_adjoints(finals, logs, g), want, atol=1e-5)
    # a decay product that underflows in the linear domain stays finite in the log domain
    tiny = [torch.full((1, 1), -60000.0), torch.full((1, 1), -0.1)]
    c = ema_dist.fold_carries([torch.ones(1, 1, 1), torch.ones(1, 1, 1)], tiny, 2)
    assert torch.isfinite(c).all()
