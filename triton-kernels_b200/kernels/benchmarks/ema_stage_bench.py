"""Per-stage benchmarks in the format of the reference's raw stage benchmarks:

    state_pass      kernels/benchmarks/ema/state_pass/state_pass_bench.py            (_ema_state_passing_fwd)
    dstates         kernels/benchmarks/ema_bwd/dstates/ema_scan_bwd_dstates_bench.py (_ema_chunk_scan_bwd_dstates)
    bwd_state_pass  kernels/benchmarks/ema_bwd/state_pass/ema_state_pass_bwd_bench.py (_ema_state_passing_bwd)
    state_fwd       the chunk-state stage (_ema_chunk_state_fwd), same byte model as dstates
    cumsum          kernels/benchmarks/ema/cumsum/cumsum_bench.py                     (ema_chunk_cumsum_fwd)
    scan_fwd        kernels/benchmarks/ema/scan_fwd/scan_fwd_bench.py                 (_ema_scan_fwd)

The reference's scan_fwd file counts only the chunk states and the cumulative sums as read and one state per chunk as
written (not x, nor the output of x's size); its figure is kept under that name, and the rate by the bytes the stage
really moves (x read, output written, cumulative sums and states read) is printed beside it.

Same shapes (fp32, B = 16, HEAD_DIM = 1024, chunk 128, SEQLEN 8192 .. 65536), same byte models (the tensors each stage
reads plus the tensors it writes, as those files count them), same outputs (a CSV per stage with one row per SEQLEN,
and a raw log line per measurement).  Timing is a CUDA-graph replay of the drop-in call, like the reference's
triton.testing.do_bench_cudagraph; this package does not depend on Triton.

    python -m kernels.benchmarks.ema_stage_bench [--seqlens 8192 ... ] [--stages state_pass dstates ...] [--out DIR]
"""
import argparse
import os

import torch

from kernels.benchmarks.ema_bench import gpu_name, time_ms_graph
from kernels.ema_kernels.ema_cumsum import ema_chunk_cumsum_fwd
from kernels.ema_kernels.ema_scan_fwd import _ema_scan_fwd
from kernels.ema_kernels.ema_state_fwd import _ema_chunk_state_fwd
from kernels.ema_kernels.ema_state_pass import _ema_state_passing_fwd
from kernels.ema_kernels_bwd.ema_scan_bwd import _ema_chunk_scan_bwd_dstates
from kernels.ema_kernels_bwd.ema_state_passing_bwd_dstates import _ema_state_passing_bwd

BATCH_SIZE = 16
MAMBA_NUM_HEADS = 2
MAMBA_CHUNK_SIZE = 128
STAGES = ("state_pass", "dstates", "bwd_state_pass", "state_fwd", "cumsum", "scan_fwd")


def _size(*tensors):
    return sum(t.numel() * t.element_size() for t in tensors)


def bench_stage(stage, BATCH, SEQLEN, HEAD_DIM, Q, device="cuda"):
    C = (SEQLEN + Q - 1) // Q
    f32 = dict(device=device, dtype=torch.float32)
    moved = None   # bytes really moved, where the reference's byte model counts something else
    if stage == "cumsum":
        P = torch.rand((BATCH, SEQLEN, 1), **f32) * 0.98 + 0.01
        A_ema = torch.log(1 - P).squeeze(-1)
        fn = lambda: ema_chunk_cumsum_fwd(A_ema, chunk_size=Q)
        bytes_moved = _size(P) + BATCH * Q * C * 4
    elif stage == "scan_fwd":
        x = torch.randn((BATCH, SEQLEN, HEAD_DIM), **f32)
        cs = -torch.rand((BATCH, C, Q), **f32).cumsum(-1)
        states = torch.randn((BATCH, C, HEAD_DIM), **f32)
        fn = lambda: _ema_scan_fwd(x, cs, states)
        bytes_moved = _size(states, cs) + BATCH * C * HEAD_DIM * 4
        moved = 2 * _size(x) + _size(states, cs)
    elif stage == "state_pass":
        states = torch.randn((BATCH, C, HEAD_DIM), **f32)
        cs_last = -torch.rand((BATCH, C), **f32)
        fn = lambda: _ema_state_passing_fwd(states, cs_last, out_dtype=torch.float32)
        bytes_moved = _size(states, cs_last) + BATCH * C * HEAD_DIM * 4
    elif stage == "bwd_state_pass":
        states = torch.randn((BATCH, C, HEAD_DIM), **f32)
        dout = torch.randn_like(states)
        dA = -torch.rand((BATCH, C), **f32)
        fn = lambda: _ema_state_passing_bwd(states, dA, dout, dfinal_states=None, seq_idx=None, has_initial_states=False,
                                            dstates_dtype=dout.dtype, states_dtype=states.dtype, chunk_size=Q)
        bytes_moved = _size(states, dA, dout) + _size(dout) + _size(dA)
    else:
        x = torch.randn((BATCH, SEQLEN, HEAD_DIM), **f32)
        cs = -torch.rand((BATCH, C, Q), **f32).cumsum(-1)
        if stage == "dstates":
            fn = lambda: _ema_chunk_scan_bwd_dstates(cs, x, dtype=torch.float32)
        else:
            fn = lambda: _ema_chunk_state_fwd(x, cs, seq_idx=None, states=None, states_in_fp32=True)
        bytes_moved = _size(x) + BATCH * C * Q * 4 + BATCH * C * HEAD_DIM * 4
    with torch.no_grad():
        ms = time_ms_graph(fn)
    if moved is not None:
        print(f"[{stage}] SEQLEN {SEQLEN}: {ms:.3f} ms, {moved / (ms * 1e-3) / 1e9:.1f} GB/s by the bytes really moved "
              f"({moved / 1e6:.1f} MB)")
    return bytes_moved / (ms * 1e-3) / 1e9, ms, bytes_moved


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--seqlens", type=int, nargs="+", default=[8192, 16384, 32768, 65536])
    ap.add_argument("--stages", nargs="+", default=list(STAGES), choices=STAGES)
    ap.add_argument("--head-dim", type=int, default=1024)
    ap.add_argument("--out", default=os.path.join(".", "kernels", "benchmarks", "outputs_ema_stages"))
    args = ap.parse_args()
    out_dir = os.path.join(args.out, gpu_name())
    os.makedirs(out_dir, exist_ok=True)
    for stage in args.stages:
        name = (f"{stage}_raw_True_time_False_ema_b{BATCH_SIZE}_chunk_size{MAMBA_CHUNK_SIZE}_head_dim{args.head_dim}"
                f"_nh{MAMBA_NUM_HEADS}.bench")
        lines = ["SEQLEN,Ema"]
        for L in args.seqlens:
            gbps, ms, nbytes = bench_stage(stage, BATCH_SIZE, L, args.head_dim, MAMBA_CHUNK_SIZE)
            lines.append(f"{float(L):.6f},{gbps:.6f}")
            with open(os.path.join(out_dir, name), "a+") as f:
                f.write("=" * 50 + stage.upper() + "=" * 50 + "\n")
                f.write(f"[ema] ms={ms:.3f}  bytes_moved={nbytes / 1e6:.3f} MB  GBps={gbps:.6f} \n")
        with open(os.path.join(out_dir, name + ".csv"), "w") as f:
            f.write("\n".join(lines) + "\n")
        print(name + " (GB/s by the reference's byte model):")
        print("\n".join(lines))


if __name__ == "__main__":
    main()
