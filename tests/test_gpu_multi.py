"""Two GPUs, one process per GPU over NCCL: row sharding and the sequence-parallel mode against the
single-GPU result.  Skipped on a box with one GPU."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _inputs(per_head, dtype):
    g = torch.Generator().manual_seed(123)
    b, L, h, d = 4, 2048, 2, 256
    x = torch.randn((b, L, h, d), generator=g).to(dtype)
    dy = torch.randn((b, L, h, d), generator=g).to(dtype)
    a = torch.sigmoid(2 + 4 * torch.rand((h,) if per_head else (b, L, h), generator=g))
    return x, a, dy


def _worker(rank, world, port, mode, per_head, dtype_name, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import ema_b200
        from ema_b200 import dist as ed
        dtype = getattr(torch, dtype_name)
        x, a, dy = _inputs(per_head, dtype)
        b, L, h, d = x.shape
        if mode == "sp":
            seg = L // world
            sl = slice(rank * seg, (rank + 1) * seg)
            xs = x[:, sl].to(dev).requires_grad_(True)
            a_s = (a if per_head else a[:, sl]).to(dev).requires_grad_(True)
            y = ed.ema_sequence_parallel(xs, a_s)
            y.backward(dy[:, sl].to(dev))
        else:
            xs, a_s = ed.shard_rows(x, a, rank, world)
            b0, b1, h0, h1 = ed.plan_row_shards(b, h, world)[rank]
            xs = xs.to(dev).requires_grad_(True)
            a_s = a_s.to(dev).requires_grad_(True)
            y = ed.ema_row_sharded(xs, a_s, heads_replicated=True)
            y.backward(dy[b0:b1, :, h0:h1].to(dev))
        torch.cuda.synchronize()
        status = ema_b200.lib().ema_b200_device_status(1)
        q.put((rank, y.detach().float().cpu().numpy(), xs.grad.float().cpu().numpy(), a_s.grad.float().cpu().numpy(), status))
    finally:
        dist.destroy_process_group()


def _single(per_head, dtype):
    import ema_b200
    x, a, dy = _inputs(per_head, dtype)
    xd = x.cuda().requires_grad_(True)
    ad = a.cuda().requires_grad_(True)
    y = ema_b200.ema(xd, ad)
    y.backward(dy.cuda())
    return y.detach().float().cpu().numpy(), xd.grad.float().cpu().numpy(), ad.grad.float().cpu().numpy()


def _run(mode, per_head, dtype_name):
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, mode, per_head, dtype_name, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = {}
    for _ in range(world):
        r, y, dx, da, status = q.get(timeout=300)
        assert status == 0
        out[r] = (y, dx, da)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    return out


@pytest.fixture(scope="module", autouse=True)
def _need_two_gpus(ema_lib):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")


@pytest.mark.parametrize("per_head", [False, True])
@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
def test_row_sharded_matches_single_gpu(per_head, dtype_name):
    out = _run("rows", per_head, dtype_name)
    y_ref, dx_ref, da_ref = _single(per_head, getattr(torch, dtype_name))
    y = np.concatenate([out[r][0] for r in range(2)], axis=0)
    dx = np.concatenate([out[r][1] for r in range(2)], axis=0)
    # the same kernels on the same rows: bitwise equal
    assert np.array_equal(y, y_ref) and np.array_equal(dx, dx_ref)
    if per_head:
        for r in range(2):
            assert np.abs(out[r][2] - da_ref).max() <= 1e-5 * np.abs(da_ref).max() + 1e-5
    else:
        da = np.concatenate([out[r][2] for r in range(2)], axis=0)
        assert np.array_equal(da, da_ref)


@pytest.mark.parametrize("per_head", [False, True])
@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
def test_sequence_parallel_matches_single_gpu(per_head, dtype_name):
    out = _run("sp", per_head, dtype_name)
    y_ref, dx_ref, da_ref = _single(per_head, getattr(torch, dtype_name))
    y = np.concatenate([out[r][0] for r in range(2)], axis=1)
    dx = np.concatenate([out[r][1] for r in range(2)], axis=1)
    tol = 1e-4 if dtype_name == "float32" else 2e-2
    assert np.abs(y - y_ref).max() <= tol * max(1.0, np.abs(y_ref).max())
    assert np.abs(dx - dx_ref).max() <= tol * max(1.0, np.abs(dx_ref).max())
    if per_head:
        for r in range(2):
            assert np.abs(out[r][2] - da_ref).max() <= tol * np.abs(da_ref).max()
    else:
        da = np.concatenate([out[r][2] for r in range(2)], axis=1)
        assert np.abs(da - da_ref).max() <= tol * np.abs(da_ref).max()
