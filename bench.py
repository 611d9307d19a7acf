#!/usr/bin/env python
"""EMA chunked scan benchmark: forward + backward tokens/s on B200, with roofline and CPU baseline.

    python bench.py [--gpus N] [--steps K] [--warmup W]            # this library
    python bench.py --impl reference [--steps K] [--warmup W]      # the reference's CPU path
    python bench.py --workload c2|c4 [--no-e2e]                    # the other single-GPU configurations
    torchrun ... bench.py --gpus N --workload c5                    # sequence parallel, one 65536-step segment per rank

One "step" is one forward (y, saved tile states) plus one backward (dx, da) over one batch of
synthetic input with the shapes of the headline workload: x, dy bf16 [16, 8192, 2, 1024] ~ N(0,1),
time-invariant decay a fp32 [2] = sigmoid(U(2,6)).  A token is one (b, t) position (all h*d
channels), so a step processes b*L = 131072 tokens per GPU.  With N > 1 every rank runs its own
batch shard of that size (rows are independent: no data-path collective; the per-head decay
gradient is all-reduced, h floats) and the reported value is the whole-job aggregate.

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
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx,
                "reasons": sorted(reasons), "samples": len(sm),
                "window": "about 1.2 s of identical back-to-back steps ending with the timed steps"}


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
    oracle/ema_loop_port.py, on a bounded sample: `b` batch rows of the workload, `L` steps."""
    import torch
    from oracle import ema_loop_port as lp
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
        "config": {"workload": WORKLOAD["name"], "sample": sample},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample,
                         "host_cpus": os.cpu_count()},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
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
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    elif WORKLOADS[args.workload].get("seq_parallel"):
        # the sequence-parallel entry point needs a process group even when it has a single member
        dist.init_process_group("nccl", store=dist.HashStore(), rank=0, world_size=1, device_id=dev)

    import ema_b200
    from ema_b200 import ops
    # one process per GPU: keep the process (and the pinned buffers of the end-to-end leg) on the GPU's NUMA node
    numa_node = ema_b200.bind_to_gpu_numa_node(dev)

    if world > 1:
        # Every step ends with a small collective that overlaps the next step's kernels.  Keep whole work items per
        # thread block (128 of the 148 SMs busy on this workload): the collective's kernel then finds a free SM
        # instead of holding back one thread block of a grid that fills the GPU.
        ema_b200.lib().ema_b200_set_split(0)
    W = WORKLOADS[args.workload]
    b, L, h, d = W["b"], W["L"], W["h"], W["d"]
    per_head, fwd_only = W["per_head"], W["fwd_only"]
    seq_parallel = bool(W.get("seq_parallel"))
    g = torch.Generator(device=dev).manual_seed(1236 + rank)
    x = torch.randn((b, L, h, d), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    dy = torch.randn((b, L, h, d), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    a_shape = (h,) if per_head else (b, L, h)
    a = torch.sigmoid(W["lo"] + (W["hi"] - W["lo"]) *
                      torch.rand(a_shape, generator=torch.Generator(device=dev).manual_seed(99), device=dev))
    y = torch.empty_like(x)
    dx = torch.empty_like(x)
    # Two buffers for the per-head decay gradient: with N > 1 its all-reduce (the only collective of the
    # row-sharded path, 4*h bytes) runs on NCCL's stream while the next step computes; a step waits for the
    # reduce issued two steps earlier before it overwrites that buffer.
    da_bufs = [torch.empty_like(a), torch.empty_like(a)]
    pending = [None, None]
    n_steps_done = 0
    ts, nt = ops.n_tiles_of(x, a)
    tile_states = torch.empty((b * h, nt, d), dtype=torch.float32, device=dev)
    ws = None
    fws = ops.ema_fwd(x, a, out=y, tile_states=tile_states)["fwd_workspace"]   # the forward's scratch, reused by every step

    def reduce_da():
        nonlocal n_steps_done
        slot = n_steps_done % 2
        n_steps_done += 1
        if world > 1 and per_head:
            pending[slot] = dist.all_reduce(da_bufs[slot], async_op=True)

    def da_slot():
        slot = n_steps_done % 2
        if pending[slot] is not None:
            pending[slot].wait()   # stream-level wait for the reduce that last used this buffer
            pending[slot] = None
        return da_bufs[slot]

    def drain():
        for slot in range(2):
            if pending[slot] is not None:
                pending[slot].wait()
                pending[slot] = None

    def sp_forward():
        from ema_b200 import dist as ema_dist
        xr, ar = x.detach().requires_grad_(True), a.detach().requires_grad_(True)
        return xr, ar, ema_dist.ema_sequence_parallel(xr, ar)

    def step():
        nonlocal ws
        if seq_parallel:
            _, _, out = sp_forward()
            out.backward(dy)
            return
        ops.ema_fwd(x, a, out=y, tile_states=tile_states, workspace=fws)
        if fwd_only:
            return
        r = ops.ema_bwd(x, a, dy, tile_states, dx=dx, ddecay=da_slot(), workspace=ws)
        ws = r["workspace"]
        reduce_da()

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()

    # Context only (not the reported value): the two calls timed alone, a few launches right after warm-up, before
    # the GPU has settled at its power-capped clock - the way the copy-bandwidth denominator itself was measured.
    burst = None
    if not seq_parallel and not fwd_only and not args.no_spinup:
        time.sleep(0.5)
        bev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(5)]
        for e in bev:
            e[0].record()
            ops.ema_fwd(x, a, out=y, tile_states=tile_states, workspace=fws)
            e[1].record()
            ops.ema_bwd(x, a, dy, tile_states, dx=dx, ddecay=da_bufs[0], workspace=ws)
            e[2].record()
        torch.cuda.synchronize()
        burst = (min(e[0].elapsed_time(e[1]) for e in bev), min(e[1].elapsed_time(e[2]) for e in bev))

    K = args.steps
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(K)]
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    # The timed region lasts tens of milliseconds, less than one nvidia-smi sample.  So that the clock
    # record describes the same load, identical steps run untimed for about a second right before it
    # (at least 5 sampler periods); the samples cover that run-in and the timed steps.
    t_begin = time.time()
    if not args.no_spinup:
        # a fixed count on every rank (each step carries a collective when N > 1): ~1.2 s at the measured step time
        t0 = time.time()
        for _ in range(20):
            step()
        torch.cuda.synchronize()
        per_step = max((time.time() - t0) / 20, 1e-5)
        n_spin = torch.tensor([int(1.2 / per_step)], device=dev)
        if world > 1:
            dist.broadcast(n_spin, 0)
        for _ in range(int(n_spin.item())):
            step()
        torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    start = torch.cuda.Event(enable_timing=True)
    stop = torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(K):
        ev[i][0].record()
        if seq_parallel:
            _, _, out = sp_forward()
            ev[i][1].record()
            out.backward(dy)
            ev[i][2].record()
            del out
            continue
        ops.ema_fwd(x, a, out=y, tile_states=tile_states, workspace=fws)
        ev[i][1].record()
        if not fwd_only:
            ops.ema_bwd(x, a, dy, tile_states, dx=dx, ddecay=da_slot(), workspace=ws)
        ev[i][2].record()
        if not fwd_only:
            reduce_da()
    drain()   # the last reduces finish inside the timed region
    stop.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t_end = time.time()
    elapsed_ms = start.elapsed_time(stop)
    if world > 1:
        t = torch.tensor([elapsed_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    clocks = sampler.stop(t_begin, t_end) if rank == 0 else None

    fwd_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in ev)
    bwd_ms = statistics.mean(e[1].elapsed_time(e[2]) for e in ev)
    ms_per_step = elapsed_ms / K
    tokens = b * L * world
    value = tokens / (ms_per_step * 1e-3)

    # ---- end to end through the public API with host buffers (pinned), copies inside the timing
    e2e = None
    try:
        if args.no_e2e:
            raise RuntimeError("skipped (--no-e2e)")
        if fwd_only:
            raise RuntimeError("skipped: the host pipeline runs forward + backward, this workload is forward only")
        if seq_parallel:
            raise RuntimeError("skipped: the host pipeline shards batch rows, this workload shards the sequence")
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
        if not torch.equal(hy, y.cpu()) or not torch.equal(hdx, dx.cpu()):
            raise RuntimeError("host pipeline result differs from the device-resident result")
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
        e2e = {"value": tokens / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": 2 * nbytes + 4 * a.numel(), "d2h_bytes_per_step": 2 * nbytes + 4 * a.numel(),
               "api": "ema_b200.HostPipeline.run(sync=False) per step + wait(): pinned host x, dy, a -> y, dx, da; "
                      "8 batch slices, H2D / kernels / D2H on three streams, consecutive steps overlap",
               "gpu_launches_per_step": pipe.n_launches, "numa_node": numa_node}
        del hx, hdy, hy, hdx, pipe
    except RuntimeError as exc:  # e.g. pinned allocation refused
        e2e = {"value": None, "unit": UNIT, "error": str(exc)[:200]}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_kind = measured_peaks()
    fwd_b, bwd_b = algorithmic_bytes(b, L, h, d, per_head=per_head)
    fwd_gbs = fwd_b / (fwd_ms * 1e-3) / 1e9
    fwd_obj = {"achieved": fwd_gbs, "frac": fwd_gbs / peak, "algorithmic_bytes_per_launch": fwd_b,
               "ms_per_launch": fwd_ms}
    if fwd_only:
        roofline = {"bound": "hbm", "kernel": "ema_fwd (scan: reads x, writes y and the saved tile states)",
                    "achieved": fwd_gbs, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": fwd_gbs / peak,
                    "traffic": None, "algorithmic_bytes_per_launch": fwd_b, "ms_per_launch": fwd_ms}
    else:
        bwd_gbs = bwd_b / (bwd_ms * 1e-3) / 1e9
        roofline = {"bound": "hbm",
                    "kernel": "ema_bwd (reverse scan: reads x, dy, writes dx; plus its small da reduction)",
                    "achieved": bwd_gbs, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                    "frac": bwd_gbs / peak, "traffic": None,
                    "algorithmic_bytes_per_launch": bwd_b, "ms_per_launch": bwd_ms, "fwd": fwd_obj,
                    "step": {"achieved": (fwd_b + bwd_b) / (ms_per_step * 1e-3) / 1e9,
                             "frac": (fwd_b + bwd_b) / (ms_per_step * 1e-3) / 1e9 / peak}}
    if burst is not None:
        roofline["timed_alone"] = {
            "fwd_ms": burst[0], "bwd_ms": burst[1], "fwd_frac": fwd_b / (burst[0] * 1e-3) / 1e9 / peak,
            "bwd_frac": bwd_b / (burst[1] * 1e-3) / 1e9 / peak,
            "note": "best of 5 launches right after warm-up, before the clocks settle under the power cap; "
                    "every other figure of this line is from the timed steps under sustained load"}
    traffic_file = os.path.join(ROOT, "profiles", "traffic.json")
    if args.workload == "c3" and os.path.exists(traffic_file):
        # dram__bytes_read.sum + dram__bytes_write.sum from the committed ncu capture of this workload
        with open(traffic_file) as f:
            tr = json.load(f)
        roofline["traffic"] = tr.get("ema_bwd_bytes_per_launch")
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
            an = a.cpu().numpy()
            t0 = time.perf_counter()
            eo.fwd(xs, an)
            eo.bwd(xs, an, xs)
            cpu_baseline["c_oracle_tokens_per_s"] = 2 * L / (time.perf_counter() - t0)
            cpu_baseline["c_oracle_threads"] = min(eo.threads(), 2 * h)
        except Exception as exc:  # the C oracle is optional context, never the measured product
            cpu_baseline["c_oracle_error"] = str(exc)[:120]

    line = {
        "metric": "ema_fwd_tokens_per_s" if fwd_only else METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16 in/out, f32 accumulate", "data": "synthetic",
        "config": {"workload": W["name"], "b_per_gpu": b, "L": L, "h": h, "d": d, "chunk": W["chunk"],
                   "tile_steps": ts,
                   "sharding": ("contiguous sequence segment per rank; all-gather of per-row carries, prefix / suffix "
                                "re-scan") if seq_parallel else "batch rows per rank, no data-path collective",
                   "decay": "per head [h]" if per_head else "per step [b, L, h]",
                   "schedule": "whole items per thread block" if world > 1 else "tiles cut evenly over the SMs",
                   "l2": f"inputs ({x.numel() * 2 * (1 if fwd_only else 2) / 2**30:.1f} GiB per step) exceed the 126 MB L2; "
                         "no flush needed"},
        "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e,
        "gpu_launches": (1 if fwd_only else 4 if per_head else 3) * K * (2 if seq_parallel and world > 1 else 1),
        "clocks": clocks,
    }
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
