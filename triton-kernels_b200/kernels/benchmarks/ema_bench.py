"""Forward EMA benchmark in the format of the reference's kernels/benchmarks/ema_bench.py.

Same providers (minus the upstream Mamba package, which is not a dependency here), same shapes (fp32, B = 16,
HEAD_DIM = 1024, two heads for the heads-style provider, chunk 128), same byte model (x read + y written + p read,
ema_bench.py:141-145), same outputs: a CSV with one row per SEQLEN and one column per provider, and a raw log per
provider and length.  Timing is a CUDA-graph replay of the call (many replays between two CUDA events), which is what the
reference's triton.testing.do_bench_cudagraph measures: the GPU time of the call without the host's launch cost; this
package does not depend on Triton.  --eager times single eager calls instead (median of CUDA-event measurements).

    python -m kernels.benchmarks.ema_bench [--seqlens 8192 16384 32768 65536] [--dtype fp32|bf16] [--out DIR]
"""
import argparse
import os
import statistics

import torch

from kernels.ema import ema_scan_combined
from kernels.ema_combined import ema_chunk_scan_combined
from kernels.ema_kernels.ema_combined_fwd import ema_matmul_scan_combined

MAMBA_NUM_HEADS = 2
MAMBA_CHUNK_SIZE = 128
PROVIDERS = [("triton_matmul", "Triton_matmul"), ("triton_prefix", "Triton Prefix"), ("ema_mamba", "Ema_mamba")]


def gpu_name():
    name = torch.cuda.get_device_name(0)
    for token in ["NVIDIA", "GeForce", "RTX", "PCIe", "GPU"]:
        name = name.replace(token, "")
    return name.strip().replace(" ", "_")


def time_ms(fn, warmup=5, reps=20):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    return statistics.median(times)


def time_ms_graph(fn, warmup=3, reps=20):
    """GPU time of one call of `fn`: the call is captured into a CUDA graph (its allocations come from the graph's own
    pool) and the graph is replayed `reps` times between two CUDA events.  Falls back to eager timing if the call cannot
    be captured."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(warmup):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    try:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
    except RuntimeError:
        torch.cuda.synchronize()
        return time_ms(fn, warmup=warmup, reps=reps)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def bench_ema(BATCH, SEQLEN, HEAD_DIM, provider, dtype, raw_dir, eager=False):
    device = "cuda"
    x = torch.randn((BATCH, SEQLEN, HEAD_DIM), dtype=torch.float32, device=device).to(dtype)
    p = torch.sigmoid(torch.randn((BATCH, SEQLEN, 1), dtype=torch.float32, device=device))
    if provider == "triton_prefix":
        fn = lambda: ema_scan_combined(x, p)
    elif provider == "ema_mamba":
        dt = -torch.log(1 - p).squeeze(-1)
        X_m = (x.float() / dt[..., None]).to(dtype).reshape(BATCH, SEQLEN, MAMBA_NUM_HEADS, HEAD_DIM // MAMBA_NUM_HEADS)
        dt = dt[..., None].expand(BATCH, SEQLEN, MAMBA_NUM_HEADS).contiguous()
        A = -torch.ones(MAMBA_NUM_HEADS, dtype=torch.float32, device=device)
        B_m = p.reshape(BATCH, SEQLEN, 1, 1)
        C_m = torch.ones_like(B_m)
        fn = lambda: ema_chunk_scan_combined(X_m, dt, A, B_m, C_m, chunk_size=MAMBA_CHUNK_SIZE, seq_idx=None)
    elif provider == "triton_matmul":
        A_ema = torch.log(1 - p).squeeze(-1)
        X_ema = (x.float() * p).to(dtype)
        fn = lambda: ema_matmul_scan_combined(A_ema, X_ema, chunk_size=MAMBA_CHUNK_SIZE)
    else:
        raise ValueError(provider)
    with torch.no_grad():
        ms = time_ms(fn) if eager else time_ms_graph(fn)
    bytes_moved = 2 * x.numel() * x.element_size() + p.numel() * p.element_size()
    gbps = bytes_moved / (ms * 1e-3) / 1e9
    raw = os.path.join(raw_dir, f"raw_{provider}_b{BATCH}_seq{SEQLEN}_chunk{MAMBA_CHUNK_SIZE}_h{HEAD_DIM}_nh{MAMBA_NUM_HEADS}.bench")
    with open(raw, "a+") as f:
        f.write("\n================= BENCHMARK RESULT =================\n")
        f.write(f"[{provider}]   ms={ms:.3f}   GB/s={gbps:.4f}\n")
        f.write(f"bytes moved = {bytes_moved/1e6:.3f} MB\n")
    return gbps, ms


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--seqlens", type=int, nargs="+", default=[8192])
    ap.add_argument("--dtype", choices=["fp32", "bf16"], default="fp32")
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--head-dim", type=int, default=1024)
    ap.add_argument("--out", default=os.path.join(".", "kernels", "benchmarks", "outputs_ema_scan"))
    ap.add_argument("--eager", action="store_true", help="time single eager calls instead of CUDA-graph replays")
    args = ap.parse_args()
    dtype = torch.float32 if args.dtype == "fp32" else torch.bfloat16
    out_dir = os.path.join(args.out, gpu_name())
    raw_dir = os.path.join(out_dir, "raw")
    os.makedirs(raw_dir, exist_ok=True)
    name = f"ema_b{args.batch}_head_dim{args.head_dim}_nh{MAMBA_NUM_HEADS}_chunk{MAMBA_CHUNK_SIZE}.bench"
    rows = []
    for L in args.seqlens:
        rows.append([float(L)] + [bench_ema(args.batch, L, args.head_dim, prov, dtype, raw_dir, args.eager)[0] for prov, _ in PROVIDERS])
    header = ",".join(["SEQLEN"] + [n for _, n in PROVIDERS])
    lines = [header] + [",".join(f"{v:.6f}" for v in r) for r in rows]
    with open(os.path.join(out_dir, name + ".csv"), "w") as f:
        f.write("\n".join(lines) + "\n")
    print(f"{name} ({args.dtype}, GB/s by the reference's byte model):")
    print("\n".join(lines))


if __name__ == "__main__":
    main()
