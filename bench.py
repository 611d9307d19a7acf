#!/usr/bin/env python
"""EMA chunked scan benchmark: forward + backward tokens/s on B200, with roofline and CPU baseline.

    python bench.py [--gpus N] [--steps K] [--warmup W]            # this library
    python bench.py --impl reference [--steps K] [--warmup W]      # the reference's CPU path
    python bench.py --workload c2|c4 [--no-e2e]                    # the other single-GPU configurations
    torchrun ... bench.py --gpus N --workload c5                    # sequence parallel only, one 65536-step segment per rank

One "step" is one forward (y, saved tile states) plus one backward (dx, da) over one batch of
synthetic input with the shapes of the headline workload: x, dy bf16 [16, 8192, 2, 1024] ~ N(0,1),
time-invariant decay a fp32 [2] = sigmoid(U(2,6)).  A token is one (b, t) position (all h*d
channels), so a step processes b*L = 131072 tokens per GPU.  With N > 1 every rank runs its own
batch shard of that size (rows are independent: no data-path collective; the per-head decay
gradient is all-reduced, h floats) and the reported value is the whole-job aggregate (weak scaling).

With N > 1 the same line also carries
  "parity"  a small-case check, on the live process group and before anything is timed, of the two multi-GPU
            modes (row sharding, sequence parallel; fp32 and bf16; per-step and per-head decay) against the
            sequential definition evaluated on the un-split tensors; the run fails when it is out of tolerance;
  "strong"  the headline batch of 16 split over the N ranks (strong scaling of the same step);
  "sp"      the sequence-parallel configuration, one 65536-step segment of b8 h4 d1024 per rank, with its
            local-scan / exchange / re-scan split and its roofline fraction.

Prints ONE JSON line on rank 0.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "triton-kernels_b200"))
sys.path.insert(0, ROOT)

# The headline workload (default) and the other single-GPU configurations of the benchmark suite.
WORKLOADS = {
    "c3": dict(name="ema_fwd_bwd_b16_L8192_h2_d1024_bf16_perhead_decay_chunk256",
               b=16, L=8192, h=2, d=1024, chunk=256, per_head=True, fwd_only=False, lo=2.0, hi=6.0),
    "c2": dict(name="ema_fwd_b16_L8192_h2_d1024_bf16_perstep_decay_chunk128",
               b=16, L=8192, h=2, d=1024, chunk=128, per_head=False, fwd_only=True, lo=2.0, hi=6.0),
    # the c2 tensors with the backward as well: the per-step decay path at a size a profiler can capture
    "c2b": dict(name="ema_fwd_bwd_b16_L8192_h2_d1024_bf16_perstep_decay_chunk128",
                b=16, L=8192, h=2, d=1024, chunk=128, per_head=False, fwd_only=False, lo=2.0, hi=6.0),
    "c4": dict(name="ema_fwd_bwd_b4_L65536_h8_d1024_bf16_perstep_decay_chunk512",
               b=4, L=65536, h=8, d=1024, chunk=512, per_head=False, fwd_only=False, lo=3.0, hi=8.0),
    # one rank's share of the headline batch when it is split over 8 GPUs (strong scaling): 4 scan rows = 32 work items,
    # the few-item case in which every row is cut into pieces that start from per-tile aggregates
    "c3_shard8": dict(name="ema_fwd_bwd_b2_L8192_h2_d1024_bf16_perhead_decay_chunk256_one_eighth_of_headline_batch",
                      b=2, L=8192, h=2, d=1024, chunk=256, per_head=True, fwd_only=False, lo=2.0, hi=6.0),
    # sequence parallel: every rank holds one contiguous 65536-step segment of b8 h4 d1024 sequences of length
    # 65536 * N (N = 8 gives the suite's 524288-step configuration); carries are exchanged over NCCL
    "c5": dict(name="ema_fwd_bwd_seqparallel_b8_Lseg65536_h4_d1024_bf16_perstep_decay_chunk256",
               b=8, L=65536, h=4, d=1024, chunk=256, per_head=False, fwd_only=False, lo=2.0, hi=6.0, seq_parallel=True),
}
WORKLOAD = WORKLOADS["c3"]
# Bounded sample of the headline workload for the CPU arms: (batch rows, steps).  About 20 s per pass.
CPU_SAMPLE = (1, 4096)
CPU_SAMPLE_NOTE = ("The loop is sequential over rows and steps, and its autograd backward pays for one full-length "
                   "gradient buffer per indexed step, so the time grows about quadratically with the length: at the "
                   "workload's full 8192 steps the reference is slower per token than on this sample.")
METRIC = "ema_fwd_bwd_tokens_per_s"
UNIT = "tokens/s"
NOMINAL_HBM_GBS = 8000.0   # the nominal figure the benchmark suite's own target is phrased against


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi sampled every 200 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.rows = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self, t_begin, t_end):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        inside = [r for (t, r) in self.rows if t_begin <= t <= t_end + 0.2] or [r for (_, r) in self.rows]
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in inside:
            try:
                sm.append(float(r[1]))
                mx = float(r[2])
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        power = []
        for r in inside:
            try:
                power.append(float(r[3]))
            except (ValueError, IndexError):
                pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx,
                "power_w": statistics.median(power) if power else None, "power_w_max": max(power) if power else None,
                "reasons": sorted(reasons), "samples": len(sm),
                "window": "about 1.2 s of identical back-to-back steps ending with the timed steps"}


def copy_probe(x, y, gpu_index):
    """A plain device-to-device copy of the forward's bytes (x -> y), measured the way the kernels are: the best of 5
    launches after idling, then the median of 30 after 1.2 s of back-to-back copies, with the SM clock and the power
    nvidia-smi reported during the run-in.  It shows what the power cap leaves a kernel that only moves the bytes."""
    import torch
    def timed(n):
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n)]
        for e0, e1 in ev:
            e0.record()
            y.copy_(x)
            e1.record()
        torch.cuda.synchronize()
        return [e0.elapsed_time(e1) for e0, e1 in ev]
    for _ in range(3):
        y.copy_(x)
    torch.cuda.synchronize()
    time.sleep(0.5)
    alone = min(timed(5))
    sampler = ClockSampler(gpu_index)
    sampler.start()
    time.sleep(0.3)
    t_begin = time.time()
    while time.time() - t_begin < 1.2:
        for _ in range(50):
            y.copy_(x)
        torch.cuda.synchronize()
    sustained = statistics.median(timed(30))
    clocks = sampler.stop(t_begin, time.time())
    nbytes = 2 * x.numel() * x.element_size()
    return {"bytes": nbytes, "alone_ms": alone, "alone_gbs": nbytes / (alone * 1e-3) / 1e9,
            "sustained_ms": sustained, "sustained_gbs": nbytes / (sustained * 1e-3) / 1e9,
            "sm_mhz": clocks.get("sm_mhz"), "power_w": clocks.get("power_w"), "power_w_max": clocks.get("power_w_max"),
            "reasons": clocks.get("reasons"),
            "note": "torch copy_ of x into y (the forward's bytes) on the same GPU right after the timed steps"}


def algorithmic_bytes(b, L, h, d, s=2, per_head=True):
    n = b * L * h * d
    na = 4 * h if per_head else 4 * b * L * h
    fwd = n * 2 * s + na                      # x read, y written, decay read
    bwd = n * 3 * s + na + na                 # x, dy read, dx written, decay read, its gradient written
    return fwd, bwd


# ---------------------------------------------------------------------------------------------
# CPU reference arm
# ---------------------------------------------------------------------------------------------
def cpu_reference_sample(b, L, h, d, steps, warmup):
    """Times the reference's CPU path (sequential PyTorch loop, autograd backward), restated in
    oracle/ema_loop_port.py, on a bounded sample: `b` batch rows of the workload, `L` steps.  Uses every host
    core torch may use (a launcher such as torchrun sets OMP_NUM_THREADS=1; that is undone here so that the
    figure does not depend on how the benchmark was started)."""
    import torch
    from oracle import ema_loop_port as lp
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    g = torch.Generator().manual_seed(1236)
    x = torch.randn((b, L, h, d), generator=g)
    dy = torch.randn((b, L, h, d), generator=g)
    a = torch.sigmoid(2 + 4 * torch.rand((h,), generator=g))
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        lp.north_star_fwd_bwd(x, a, dy)
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    sec = sum(times) / len(times)
    return b * L / sec, sec, torch.get_num_threads()


SCHEDULES = {0: "whole work items (scan row x 128 channels) per thread block",
             1: "tile ranges over the SMs, carries handed between thread blocks",
             2: "per-tile aggregates, then pieces of items dealt evenly over the SMs"}


def workload_config(W, schedule, tile_steps=128):
    """The `config` object of a result line: the same for this library's arm and for the reference arm."""
    b, L, h, d = W["b"], W["L"], W["h"], W["d"]
    return {"workload": W["name"], "b_per_gpu": b, "L": L, "h": h, "d": d, "chunk": W["chunk"],
            "tile_steps": tile_steps,
            "sharding": "batch rows per rank, no data-path collective",
            "decay": "per head [h]" if W["per_head"] else "per step [b, L, h]",
            "schedule": SCHEDULES.get(schedule, "cuda cores"),
            "l2": (f"tensors touched per step ({b * L * h * d * 2 * (2 if W['fwd_only'] else 4) / 2**20:.0f} MiB) exceed the "
                   "126 MB L2; no flush needed")}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sb, sL = CPU_SAMPLE
    val, sec, threads = cpu_reference_sample(sb, sL, WORKLOAD["h"], WORKLOAD["d"], args.steps, args.warmup)
    sample = (f"{sb} of {WORKLOAD['b']} batch rows x first {sL} of {WORKLOAD['L']} steps x all "
              f"{WORKLOAD['h']}x{WORKLOAD['d']} channels per step, fwd + autograd bwd. " + CPU_SAMPLE_NOTE)
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        # this library's arm's config for the same workload (its kernels run the headline on whole work items); what the
        # reference arm actually timed is in `sample`
        "config": workload_config(WORKLOAD, 0),
        "sample": sample,
        "note": "the reference checkout does not travel to the GPU box: this is the port of its sequential loop "
                "(oracle/ema_loop_port.py, pinned against the reference's own loop by the test fixtures), on the host "
                "cores, the same whatever --gpus says",
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample,
                         "host_cpus": os.cpu_count()},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------
# multi-GPU parity self-check (N > 1): both modes against the sequential definition on the un-split tensors
# ---------------------------------------------------------------------------------------------
PARITY_TOL = {"fp32_abs": 1e-4, "fp32_da": "1e-4 + 2e-5 * max|ref|", "bf16_rel": 2e-2}


def _parity_inputs(seed, b, L, h, d, per_head, dtype, lo, hi):
    import torch
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((b, L, h, d), generator=g).to(dtype)
    dy = torch.randn((b, L, h, d), generator=g).to(dtype)
    a = torch.sigmoid(lo + (hi - lo) * torch.rand((h,) if per_head else (b, L, h), generator=g))
    return x, a, dy


def multi_gpu_parity(dev, rank, world):
    """Runs ema_sequence_parallel and ema_row_sharded (forward + backward) on small seeded problems over the live
    process group, gathers the pieces on rank 0 and compares them there with the C restatement of the reference's
    sequential loop (the checker; it is never what is timed) evaluated on the whole, un-split tensors - and the
    row-sharded pieces, in addition, bit for bit with this library's own single-GPU result.  Long-memory decays
    sigmoid(U(3,8)): a carry survives several 1024-step segments, so the exchange is what is being tested."""
    import numpy as np
    import torch
    import torch.distributed as dist
    import ema_b200
    from ema_b200 import dist as ed

    def gather(t, dim):
        t = t.detach().float().contiguous()
        out = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(out, t)
        return torch.cat(out, dim=dim).cpu().numpy() if rank == 0 else None

    res = {"sp_max_err": {}, "rows_max_err": {}, "rows_bitwise": True, "tol": PARITY_TOL, "ok": True,
           "sp_shape": None, "rows_shape": None, "decay": "sigmoid(U(3,8))", "cases": 0}
    eo = None
    if rank == 0:
        from oracle import ema_oracle as eo   # checker only

    def judge(kind, name, got, ref, dtype, is_da):
        err = float(np.abs(got - ref).max())
        scale = float(np.abs(ref).max())
        if dtype == torch.float32:
            tol = 1e-4 + (2e-5 * scale if is_da else 0.0)
            shown = err
        else:
            tol = 2e-2 * max(scale, 1e-6)
            shown = err / max(scale, 1e-6)
        key = f"{'fp32' if dtype == torch.float32 else 'bf16'}_{name}"
        res[kind][key] = max(res[kind].get(key, 0.0), shown)
        if not err <= tol:
            res["ok"] = False
            sys.stderr.write(f"parity FAILED: {kind} {key}: err {err:.3e} > tol {tol:.3e}\n")

    for dtype in (torch.float32, torch.bfloat16):
        for per_head in (False, True):
            # ---- sequence parallel: b2, one 1024-step segment per rank
            b, h, d, seg = 2, 2, 128, 1024
            L = seg * world
            res["sp_shape"] = [b, L, h, d]
            x, a, dy = _parity_inputs(4000 + int(per_head), b, L, h, d, per_head, dtype, 3.0, 8.0)
            sl = slice(rank * seg, (rank + 1) * seg)
            xs = x[:, sl].to(dev).requires_grad_(True)
            a_s = (a if per_head else a[:, sl]).to(dev).requires_grad_(True)
            y = ed.ema_sequence_parallel(xs, a_s)
            y.backward(dy[:, sl].to(dev))
            gy, gdx = gather(y, 1), gather(xs.grad, 1)
            gda = a_s.grad.detach().float().cpu().numpy() if per_head else gather(a_s.grad, 1)
            if rank == 0:
                xn, an, dyn = x.float().numpy(), a.numpy(), dy.float().numpy()
                y_ref = eo.fwd(xn, an, acc64=True)
                dx_ref, da_ref = eo.bwd(xn, an, dyn, acc64=True)
                judge("sp_max_err", "y", gy, y_ref, dtype, False)
                judge("sp_max_err", "dx", gdx, dx_ref, dtype, False)
                judge("sp_max_err", "da", gda, da_ref, dtype, True)
            # ---- row sharding: one batch row per rank
            b, L = world, 1024
            res["rows_shape"] = [b, L, h, d]
            x, a, dy = _parity_inputs(5000 + int(per_head), b, L, h, d, per_head, dtype, 3.0, 8.0)
            xs, a_s = ed.shard_rows(x, a, rank, world)
            b0, b1, h0, h1 = ed.plan_row_shards(b, h, world)[rank]
            xs = xs.to(dev).requires_grad_(True)
            a_s = a_s.to(dev).requires_grad_(True)
            y = ed.ema_row_sharded(xs, a_s, heads_replicated=True)
            y.backward(dy[b0:b1, :, h0:h1].to(dev))
            gy, gdx = gather(y, 0), gather(xs.grad, 0)
            gda = a_s.grad.detach().float().cpu().numpy() if per_head else gather(a_s.grad, 0)
            if rank == 0:
                xn, an, dyn = x.float().numpy(), a.numpy(), dy.float().numpy()
                y_ref = eo.fwd(xn, an, acc64=True)
                dx_ref, da_ref = eo.bwd(xn, an, dyn, acc64=True)
                judge("rows_max_err", "y", gy, y_ref, dtype, False)
                judge("rows_max_err", "dx", gdx, dx_ref, dtype, False)
                judge("rows_max_err", "da", gda, da_ref, dtype, True)
                # the same kernels on the same rows: the pieces equal the single-GPU result bit for bit
                xd, ad = x.to(dev).requires_grad_(True), a.to(dev).requires_grad_(True)
                y1 = ema_b200.ema(xd, ad)
                y1.backward(dy.to(dev))
                same = (np.array_equal(gy, y1.detach().float().cpu().numpy()) and
                        np.array_equal(gdx, xd.grad.float().cpu().numpy()))
                if not per_head:
                    same = same and np.array_equal(gda, ad.grad.float().cpu().numpy())
                if not same:
                    res["rows_bitwise"] = False
                    res["ok"] = False
                    sys.stderr.write(f"parity FAILED: row-sharded pieces differ from the single-GPU result "
                                     f"({dtype}, per_head={per_head})\n")
            res["cases"] += 2
    torch.cuda.synchronize()
    status = ema_b200.lib().ema_b200_device_status(1)
    flag = torch.tensor([1 if (res["ok"] and status == 0) else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    res["ok"] = bool(flag.item())
    res["device_status"] = status
    return res


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
class RowShardedRun:
    """The row-sharded step (forward + backward on this rank's batch rows, plus the all-reduce of the per-head
    decay gradient when N > 1) with its buffers; used for the headline (weak scaling) and the strong-scaling runs."""

    def __init__(self, W, b_local, dev, rank, world):
        import torch
        from ema_b200 import ops
        self.torch, self.ops, self.world = torch, ops, world
        b, L, h, d = b_local, W["L"], W["h"], W["d"]
        self.shape = (b, L, h, d)
        self.per_head, self.fwd_only = W["per_head"], W["fwd_only"]
        g = torch.Generator(device=dev).manual_seed(1236 + rank)
        self.x = torch.randn((b, L, h, d), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
        self.dy = torch.randn((b, L, h, d), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
        a_shape = (h,) if self.per_head else (b, L, h)
        self.a = torch.sigmoid(W["lo"] + (W["hi"] - W["lo"]) *
                               torch.rand(a_shape, generator=torch.Generator(device=dev).manual_seed(99), device=dev))
        self.y = torch.empty_like(self.x)
        self.dx = torch.empty_like(self.x)
        # Two buffers for the per-head decay gradient: with N > 1 its all-reduce (the only collective of the
        # row-sharded path, 4*h bytes) runs on NCCL's stream while the next step computes; a step waits for the
        # reduce issued two steps earlier before it overwrites that buffer.
        self.da_bufs = [torch.empty_like(self.a), torch.empty_like(self.a)]
        self.pending = [None, None]
        self.n_done = 0
        self.tile_steps, nt = ops.n_tiles_of(self.x, self.a)
        self.tile_states = torch.empty((b * h, nt, d), dtype=torch.float32, device=dev)
        self.ws = None
        self.fws = ops.ema_fwd(self.x, self.a, out=self.y, tile_states=self.tile_states)["fwd_workspace"]

    def _reduce_da(self):
        import torch.distributed as dist
        slot = self.n_done % 2
        self.n_done += 1
        if self.world > 1 and self.per_head:
            self.pending[slot] = dist.all_reduce(self.da_bufs[slot], async_op=True)

    def _da_slot(self):
        slot = self.n_done % 2
        if self.pending[slot] is not None:
            self.pending[slot].wait()   # stream-level wait for the reduce that last used this buffer
            self.pending[slot] = None
        return self.da_bufs[slot]

    def drain(self):
        for slot in range(2):
            if self.pending[slot] is not None:
                self.pending[slot].wait()
                self.pending[slot] = None

    def fwd(self):
        self.ops.ema_fwd(self.x, self.a, out=self.y, tile_states=self.tile_states, workspace=self.fws)

    def bwd(self):
        r = self.ops.ema_bwd(self.x, self.a, self.dy, self.tile_states, dx=self.dx, ddecay=self._da_slot(),
                             workspace=self.ws)
        self.ws = r["workspace"]

    def step(self, ev=None):
        if ev:
            ev[0].record()
        self.fwd()
        if ev:
            ev[1].record()
        if not self.fwd_only:
            self.bwd()
        if ev:
            ev[2].record()
        if not self.fwd_only:
            self._reduce_da()


def timed_steps(run, K, dev, world, spin_seconds=1.2):
    """Untimed run-in of identical steps (so that clock samples describe the same load), then exactly K steps between
    CUDA events with a barrier + synchronize on both sides; the step time is the maximum over the ranks."""
    import torch
    import torch.distributed as dist
    if spin_seconds > 0:
        # a fixed count on every rank (each step carries a collective when N > 1)
        t0 = time.time()
        for _ in range(20):
            run.step()
        torch.cuda.synchronize()
        per_step = max((time.time() - t0) / 20, 1e-5)
        n_spin = torch.tensor([int(spin_seconds / per_step)], device=dev)
        if world > 1:
            dist.broadcast(n_spin, 0)
        for _ in range(int(n_spin.item())):
            run.step()
        torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(K)]
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(K):
        run.step(ev[i])
    run.drain()   # the last reduces finish inside the timed region
    stop.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    own_ms = start.elapsed_time(stop) / K
    fwd_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in ev)
    bwd_ms = statistics.mean(e[1].elapsed_time(e[2]) for e in ev)
    gap_ms = statistics.mean(ev[i][2].elapsed_time(ev[i + 1][0]) for i in range(K - 1)) if K > 1 else 0.0
    ms = own_ms
    if world > 1:
        t = torch.tensor([own_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return {"ms_per_step": ms, "own_ms_per_step": own_ms, "fwd_ms": fwd_ms, "bwd_ms": bwd_ms, "gap_ms": gap_ms}


def per_rank_table(stats, sm_mhz, dev, world):
    """min / median / max over the ranks of each rank's own figures (rank 0 returns the table)."""
    import torch
    import torch.distributed as dist
    keys = ["own_ms_per_step", "fwd_ms", "bwd_ms", "gap_ms"]
    mine = torch.tensor([stats[k] for k in keys] + [float(sm_mhz or 0.0)], device=dev, dtype=torch.float64)
    allv = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(allv, mine)
    rows = torch.stack(allv).cpu()
    out = {}
    for i, k in enumerate(keys + ["sm_mhz"]):
        col = rows[:, i]
        out[k] = {"min": float(col.min()), "median": float(col.median()), "max": float(col.max())}
    out["slowest_rank"] = int(rows[:, 0].argmax())
    out["note"] = ("every rank's own CUDA-event figures for the timed steps: fwd and bwd calls, the gap between a "
                   "backward's end and the next forward's start, and the median SM clock nvidia-smi reported for "
                   "that rank's GPU meanwhile; the step time reported is the slowest rank's")
    return out


def run_seq_parallel(W, dev, rank, world, K, peak):
    """The sequence-parallel configuration: one contiguous segment per rank, carries exchanged over NCCL."""
    import torch
    import torch.distributed as dist
    from ema_b200 import dist as ema_dist
    b, L, h, d = W["b"], W["L"], W["h"], W["d"]
    g = torch.Generator(device=dev).manual_seed(4321 + rank)
    x = torch.randn((b, L, h, d), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    dy = torch.randn((b, L, h, d), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    a = torch.sigmoid(W["lo"] + (W["hi"] - W["lo"]) * torch.rand((b, L, h), generator=g, device=dev))

    def step():
        xr, ar = x.detach().requires_grad_(True), a.detach().requires_grad_(True)
        out = ema_dist.ema_sequence_parallel(xr, ar)
        out.backward(dy)

    for _ in range(3):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ema_dist.trace = []
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(K):
        step()
    stop.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    marks, ema_dist.trace = ema_dist.trace, None
    own_ms = start.elapsed_time(stop) / K
    t = torch.tensor([own_ms], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    # stage split from the events the sequence-parallel function recorded (this rank's)
    seg = {}
    order = ["fwd_begin", "fwd_local", "fwd_exchange", "fwd_end", "bwd_begin", "bwd_local", "bwd_exchange", "bwd_end"]
    per_step = len(marks) // K if K else 0
    for s in range(K):
        chunk = dict(marks[s * per_step:(s + 1) * per_step])
        for lo, hi, name in (("fwd_begin", "fwd_local", "fwd_local_scan_ms"), ("fwd_local", "fwd_exchange", "fwd_exchange_ms"),
                             ("fwd_exchange", "fwd_end", "fwd_rescan_ms"), ("bwd_begin", "bwd_local", "bwd_local_scan_ms"),
                             ("bwd_local", "bwd_exchange", "bwd_exchange_ms"), ("bwd_exchange", "bwd_end", "bwd_rescan_ms")):
            if lo in chunk and hi in chunk:
                seg.setdefault(name, []).append(chunk[lo].elapsed_time(chunk[hi]))
    split = {k: statistics.mean(v) for k, v in seg.items()}
    del order
    if world > 1:
        # exchange and re-scan times differ by rank (rank 0 re-scans nothing in the forward): report the slowest
        keys = sorted(split)
        tt = torch.tensor([split[k] for k in keys], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        split = {k: float(v) for k, v in zip(keys, tt.cpu())}
    fwd_b, bwd_b = algorithmic_bytes(b, L, h, d, per_head=False)
    gbs = (fwd_b + bwd_b) / (ms * 1e-3) / 1e9
    local_ms = split.get("fwd_local_scan_ms", 0.0) + split.get("bwd_local_scan_ms", 0.0)
    return {"workload": W["name"], "n_ranks": world, "total_L": L * world, "steps": K, "ms_per_step": ms,
            "value": b * L * world / (ms * 1e-3), "unit": UNIT,
            "split_ms_max_over_ranks": split,
            "roofline": {"achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                         "frac_of_nominal_8TBs": gbs / NOMINAL_HBM_GBS,
                         "algorithmic_bytes_per_rank_step": fwd_b + bwd_b,
                         "local_scans_only_frac": ((fwd_b + bwd_b) / (local_ms * 1e-3) / 1e9 / peak) if local_ms else None},
            "exchange_bytes_per_rank_per_direction": b * h * (d + 1) * 4,
            "note": "per rank: local scan from a zero state, one all-gather of [final state | summed log decay] per "
                    "direction, a fold kernel, and a re-scan of the prefix (forward) / suffix (backward) that the "
                    "incoming carry still changes; value = tokens of all ranks / slowest rank's step time"}


def run_gpu(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the EMA library has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    W = WORKLOADS[args.workload]
    seq_parallel = bool(W.get("seq_parallel"))
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    elif seq_parallel:
        # the sequence-parallel entry point needs a process group even when it has a single member
        dist.init_process_group("nccl", store=dist.HashStore(), rank=0, world_size=1, device_id=dev)

    import ema_b200
    # one process per GPU: keep the process (and the pinned buffers of the end-to-end leg) on the GPU's NUMA node
    numa_node = ema_b200.bind_to_gpu_numa_node(dev)
    peak, peak_kind = measured_peaks()
    K = args.steps

    if seq_parallel:
        sp = run_seq_parallel(W, dev, rank, world, K, peak)
        if rank == 0:
            line = {"metric": METRIC, "value": sp["value"], "unit": UNIT, "n_gpus": world, "steps": K,
                    "warmup": 3, "ms_per_step": sp["ms_per_step"], "higher_is_better": True, "scaling": "weak",
                    "vs_baseline": None, "dtype": "bf16 in/out, f32 accumulate", "data": "synthetic",
                    "config": {"workload": W["name"], "b": W["b"], "L_per_rank": W["L"], "h": W["h"], "d": W["d"]},
                    "roofline": dict(sp["roofline"], bound="hbm", peak_kind=peak_kind, traffic=None), "sp": sp,
                    "cpu_baseline": None, "e2e": None, "gpu_launches": 6 * K}
            print(json.dumps(line))
        dist.destroy_process_group()
        return

    # ---- N > 1: parity of the two multi-GPU modes on the live process group, before anything is timed
    parity = None
    if world > 1 and not args.no_parity:
        parity = multi_gpu_parity(dev, rank, world)
        if not parity["ok"]:
            if rank == 0:
                print(json.dumps({"metric": METRIC, "value": None, "n_gpus": world, "parity": parity,
                                  "error": "multi-GPU parity check out of tolerance"}))
            dist.destroy_process_group()
            raise SystemExit(1)

    # (The headline workload's 256 work items run as whole items, two per thread block on 128 of the 148 SMs, at every
    # N: with N > 1 the small collective that ends a step overlaps the next step's kernels and finds a free SM.)
    b, L, h, d = W["b"], W["L"], W["h"], W["d"]
    per_head, fwd_only = W["per_head"], W["fwd_only"]
    run = RowShardedRun(W, b, dev, rank, world)
    ts = run.tile_steps
    for _ in range(max(args.warmup, 3)):
        run.step()
    run.drain()
    torch.cuda.synchronize()

    # Context only (not the reported value): the two calls timed alone, a few launches right after warm-up, before
    # the GPU has settled at its power-capped clock - the way the copy-bandwidth denominator itself was measured.
    burst = None
    if not fwd_only and not args.no_spinup:
        time.sleep(0.5)
        bev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(5)]
        for e in bev:
            e[0].record()
            run.fwd()
            e[1].record()
            run.bwd()
            e[2].record()
        torch.cuda.synchronize()
        burst = (min(e[0].elapsed_time(e[1]) for e in bev), min(e[1].elapsed_time(e[2]) for e in bev))

    # The timed region lasts tens of milliseconds, less than one nvidia-smi sample.  So that the clock record describes
    # the same load, identical steps run untimed for about a second right before it (at least 5 sampler periods); the
    # samples cover that run-in and the timed steps.  Every rank samples its own GPU.
    sampler = ClockSampler(local)
    sampler.start()
    time.sleep(0.3)
    t_begin = time.time()
    stats = timed_steps(run, K, dev, world, spin_seconds=0.0 if args.no_spinup else 1.2)
    t_end = time.time()
    clocks = sampler.stop(t_begin, t_end)
    schedule = ema_b200.lib().ema_b200_last_schedule()   # of the timed steps' last call (the backward, or the forward)
    ms_per_step, fwd_ms, bwd_ms = stats["ms_per_step"], stats["fwd_ms"], stats["bwd_ms"]
    tokens = b * L * world
    value = tokens / (ms_per_step * 1e-3)
    per_rank = per_rank_table(stats, clocks.get("sm_mhz"), dev, world) if world > 1 else None

    probe = None
    if world == 1 and not args.no_spinup and not args.no_copy_probe:
        probe = copy_probe(run.x, run.y, local)
        run.fwd()   # y holds the forward's result again
        torch.cuda.synchronize()

    # ---- strong scaling (N > 1): the headline batch split over the ranks
    strong = None
    if world > 1 and not fwd_only and b % world == 0 and not args.no_strong:
        srun = RowShardedRun(W, b // world, dev, rank, world)
        for _ in range(5):
            srun.step()
        srun.drain()
        torch.cuda.synchronize()
        s_stats = timed_steps(srun, K, dev, world, spin_seconds=0.0 if args.no_spinup else 0.4)
        s_rank = per_rank_table(s_stats, None, dev, world)
        fb, bb = algorithmic_bytes(b // world, L, h, d, per_head=per_head)
        strong = {"value": b * L / (s_stats["ms_per_step"] * 1e-3), "unit": UNIT, "ms_per_step": s_stats["ms_per_step"],
                  "global_batch": b, "b_per_gpu": b // world, "scan_rows_per_gpu": (b // world) * h,
                  "work_items_per_gpu": (b // world) * h * ((d + 127) // 128),
                  "fwd_ms": s_stats["fwd_ms"], "bwd_ms": s_stats["bwd_ms"],
                  "per_gpu_frac_of_peak": (fb + bb) / (s_stats["ms_per_step"] * 1e-3) / 1e9 / peak,
                  "whole_batch_on_one_gpu_ms_same_run": ms_per_step,
                  "speedup_over_one_gpu_same_run": ms_per_step / s_stats["ms_per_step"],
                  "per_rank": {k: s_rank[k] for k in ("own_ms_per_step", "fwd_ms", "bwd_ms")},
                  "note": "the same step with the batch of 16 split over the ranks (total work fixed); "
                          "whole_batch_on_one_gpu_ms_same_run is this line's own ms_per_step (every rank of the weak "
                          "run holds the whole batch of 16)"}
        del srun
        torch.cuda.empty_cache()

    # ---- end to end through the public API with host buffers (pinned), copies inside the timing
    e2e = None
    try:
        if args.no_e2e:
            raise RuntimeError("skipped (--no-e2e)")
        if fwd_only:
            raise RuntimeError("skipped: the host pipeline runs forward + backward, this workload is forward only")
        x, dy, a, y, dx = run.x, run.dy, run.a, run.y, run.dx
        hx, hdy = x.cpu().pin_memory(), dy.cpu().pin_memory()
        ha = a.cpu().pin_memory()
        hy, hdx = torch.empty_like(hx).pin_memory(), torch.empty_like(hx).pin_memory()
        hda = torch.empty_like(ha).pin_memory()
        # the library's host-buffer entry: batch slices stream through H2D copy, kernels and D2H copy concurrently
        pipe = ema_b200.HostPipeline((b, L, h, d), torch.bfloat16, per_head=per_head, device=dev, slices=8, depth=3)

        def e2e_step():
            pipe.run(hx, ha, hdy, hy, hdx, hda, sync=False)

        e2e_steps = min(K, 5)
        e2e_step()
        pipe.wait()
        torch.cuda.synchronize()
        # Against the device-resident result.  The pipeline's batch slices are problems with few work items, which the
        # kernels cut into pieces that start from per-tile aggregates, while the whole batch runs item by item: the two
        # agree to within the rounding of the bf16 decay matrices, not bit for bit.
        e2e_err = max(float((hy.float() - y.cpu().float()).abs().max() / y.float().abs().max()),
                      float((hdx.float() - dx.cpu().float()).abs().max() / dx.float().abs().max()))
        if not e2e_err <= 2e-2:
            raise RuntimeError(f"host pipeline result differs from the device-resident result ({e2e_err:.3e})")
        if world > 1:
            dist.barrier()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(e2e_steps):
            e2e_step()          # queued back to back: a step's first copies overlap the previous step's last ones
        pipe.wait()
        s1.record()
        torch.cuda.synchronize()
        e2e_ms = s0.elapsed_time(s1) / e2e_steps
        if world > 1:
            t = torch.tensor([e2e_ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_ms = float(t.item())
        nbytes = x.numel() * 2
        each_way = 2 * nbytes + 4 * a.numel()
        e2e = {"value": tokens / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": each_way, "d2h_bytes_per_step": each_way,
               "api": "ema_b200.HostPipeline.run(sync=False) per step + wait(): pinned host x, dy, a -> y, dx, da; "
                      "8 batch slices, H2D / kernels / D2H on three streams, consecutive steps overlap",
               "gpu_launches_per_step": pipe.n_launches, "numa_node": numa_node,
               "max_rel_diff_vs_device_resident": e2e_err,
               "host_link_gbs_each_way_all_ranks": each_way * world / (e2e_ms * 1e-3) / 1e9,
               "limit": "host-to-device and device-to-host copies (PCIe and host memory), not the kernels: all ranks "
                        "of the node share one host, so with N > 1 the aggregate copy rate each way "
                        "(host_link_gbs_each_way_all_ranks) is what the host sustains in total, and the per-rank "
                        "step time grows with N"}
        del hx, hdy, hy, hdx, pipe
    except RuntimeError as exc:  # e.g. pinned allocation refused
        e2e = {"value": None, "unit": UNIT, "error": str(exc)[:200]}

    # ---- N > 1: the sequence-parallel configuration (one 65536-step segment per rank)
    sp = None
    if world > 1 and args.workload == "c3" and not args.no_sp:
        del run
        torch.cuda.empty_cache()
        sp = run_seq_parallel(WORKLOADS["c5"], dev, rank, world, min(K, 10), peak)
        run = None

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    fwd_b, bwd_b = algorithmic_bytes(b, L, h, d, per_head=per_head)
    fwd_gbs = fwd_b / (fwd_ms * 1e-3) / 1e9
    fwd_obj = {"achieved": fwd_gbs, "frac": fwd_gbs / peak, "frac_of_nominal_8TBs": fwd_gbs / NOMINAL_HBM_GBS,
               "algorithmic_bytes_per_launch": fwd_b, "ms_per_launch": fwd_ms}
    if fwd_only:
        roofline = {"bound": "hbm", "kernel": "ema_fwd (scan: reads x, writes y and the saved tile states)",
                    "achieved": fwd_gbs, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": fwd_gbs / peak,
                    "frac_of_nominal_8TBs": fwd_gbs / NOMINAL_HBM_GBS,
                    "traffic": None, "algorithmic_bytes_per_launch": fwd_b, "ms_per_launch": fwd_ms}
    else:
        bwd_gbs = bwd_b / (bwd_ms * 1e-3) / 1e9
        step_gbs = (fwd_b + bwd_b) / (ms_per_step * 1e-3) / 1e9
        roofline = {"bound": "hbm",
                    "kernel": "ema_bwd (reverse scan: reads x, dy, writes dx; plus its small da reduction)",
                    "achieved": bwd_gbs, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                    "frac": bwd_gbs / peak, "frac_of_nominal_8TBs": bwd_gbs / NOMINAL_HBM_GBS, "traffic": None,
                    "algorithmic_bytes_per_launch": bwd_b, "ms_per_launch": bwd_ms, "fwd": fwd_obj,
                    "step": {"achieved": step_gbs, "frac": step_gbs / peak,
                             "frac_of_nominal_8TBs": step_gbs / NOMINAL_HBM_GBS}}
    if clocks.get("sm_mhz"):
        # time x clock: separates what the power-capped SM clock costs from what the kernel costs
        roofline["ms_x_sm_ghz"] = {"fwd": fwd_ms * clocks["sm_mhz"] / 1e3,
                                   "bwd": (bwd_ms * clocks["sm_mhz"] / 1e3) if not fwd_only else None}
    if burst is not None:
        roofline["timed_alone"] = {
            "fwd_ms": burst[0], "bwd_ms": burst[1], "fwd_frac": fwd_b / (burst[0] * 1e-3) / 1e9 / peak,
            "bwd_frac": bwd_b / (burst[1] * 1e-3) / 1e9 / peak,
            "note": "best of 5 launches right after warm-up, before the clocks settle under the power cap; "
                    "every other figure of this line is from the timed steps under sustained load"}
    if probe is not None:
        roofline["copy_probe"] = probe
    traffic_file = os.path.join(ROOT, "profiles", "traffic.json")
    if args.workload == "c3" and os.path.exists(traffic_file):
        # dram__bytes_read.sum + dram__bytes_write.sum from the committed ncu capture of this workload
        # (a constant read from that file, not measured in this run)
        with open(traffic_file) as f:
            tr = json.load(f)
        roofline["traffic"] = tr.get("ema_bwd_bytes_per_launch")
        roofline["traffic_source"] = "profiles/traffic.json (ncu capture of this workload), not measured in this run"
        roofline["fwd"]["traffic"] = tr.get("ema_fwd_bytes_per_launch")

    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline and args.workload == "c3":
        sb, sL = CPU_SAMPLE
        val, sec, threads = cpu_reference_sample(sb, sL, h, d, steps=1, warmup=0)
        cpu_baseline = {"value": val, "unit": UNIT, "cores": threads, "kind": "port",
                        "sample": f"{sb} of {b} batch rows x first {sL} of {L} steps, fwd + autograd bwd, "
                                  f"{sec:.1f} s. " + CPU_SAMPLE_NOTE,
                        "host_cpus": os.cpu_count()}
        try:
            from oracle import ema_oracle as eo
            import numpy as np
            xs = np.random.RandomState(0).standard_normal((2, L, h, d)).astype(np.float32)
            an = np.random.RandomState(1).uniform(0.9, 0.99, (h,)).astype(np.float32)
            t0 = time.perf_counter()
            eo.fwd(xs, an)
            eo.bwd(xs, an, xs)
            cpu_baseline["c_oracle_tokens_per_s"] = 2 * L / (time.perf_counter() - t0)
            cpu_baseline["c_oracle_threads"] = min(eo.threads(), 2 * h)
        except Exception as exc:  # the C oracle is optional context, never the measured product
            cpu_baseline["c_oracle_error"] = str(exc)[:120]

    launches_per_step = 1 if fwd_only else 3   # forward scan, backward scan, decay-gradient reduction
    if schedule == 2:
        launches_per_step += 1 if fwd_only else 2   # the aggregate passes over x and dy
    line = {
        "metric": "ema_fwd_tokens_per_s" if fwd_only else METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16 in/out, f32 accumulate", "data": "synthetic",
        "config": workload_config(W, schedule, ts),
        "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e,
        "gpu_launches": launches_per_step * K,
        "clocks": clocks,
    }
    if parity is not None:
        line["parity"] = parity
    if per_rank is not None:
        line["per_rank"] = per_rank
    if strong is not None:
        line["strong"] = strong
    if sp is not None:
        line["sp"] = sp
    print(json.dumps(line))
    if dist.is_initialized():
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c3", choices=sorted(WORKLOADS),
                    help="c3 = the headline configuration (default); c2, c4 = the other single-GPU configurations; "
                         "c5 = sequence parallel over the ranks")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg (profiling runs)")
    ap.add_argument("--no-spinup", action="store_true", help="skip the untimed run-in used for clock sampling (profiling runs)")
    ap.add_argument("--no-copy-probe", action="store_true", help="skip the plain-copy comparison (N = 1)")
    ap.add_argument("--no-parity", action="store_true", help="N > 1: skip the multi-GPU parity self-check")
    ap.add_argument("--no-strong", action="store_true", help="N > 1: skip the strong-scaling leg")
    ap.add_argument("--no-sp", action="store_true", help="N > 1: skip the sequence-parallel leg")
    args = ap.parse_args()
    if args.impl == "reference":
        # each step is one ~20 s pass over the CPU sample: keep the whole run within a few minutes
        args.steps = max(1, min(args.steps, 4))
        args.warmup = max(0, min(args.warmup, 1))
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
