"""Multi-GPU EMA: one process per GPU, torch.distributed (NCCL over NVLink) for the plumbing.

Two modes, neither of which exists in the reference project (it is single-GPU):

* row sharding - the scan rows (b, h) are independent, so every rank scans its own slice with no
  data-path collective.  Only a time-invariant decay a[h] needs one all-reduce of h floats for its
  gradient.
* sequence parallel - rank g holds the g-th contiguous segment of the sequence.  Every rank scans
  its segment from a zero state, the ranks all-gather one record each - the per-row final state
  F[b,h,d] followed by the summed log-decay logP[b,h] (kept in the log domain: the product of 65536
  decays underflows), written by the scan kernel straight into the send buffer - each rank folds
  its predecessors into its incoming carry (one small kernel), and a fix-up pass re-scans only the prefix of
  the segment that the carry can still influence.  The backward mirrors it right to left with the
  adjoint carry.  Remote data always arrives in local memory through the collective before a kernel
  reads it.

`backend` is the module providing ema_fwd / ema_bwd (default: the CUDA ops); the CPU tests pass a
stand-in so that the exchange logic runs under gloo without a GPU.
"""
import torch
import torch.distributed as dist

from . import ops as _cuda_ops

STOP_BELOW = 1e-12  # a carry attenuated below this no longer changes an fp32 result

# Timing hook for benchmarks: set to a list and the sequence-parallel function appends (label, CUDA event) at its
# stage boundaries (local scan / exchange and fold / re-scan), recorded on the current stream.  None: no events.
trace = None


def _mark(label, t):
    if trace is not None and t.is_cuda:
        ev = torch.cuda.Event(enable_timing=True)
        ev.record(torch.cuda.current_stream(t.device))
        trace.append((label, ev))


# ---- row sharding -----------------------------------------------------------------------------

def plan_row_shards(b, h, world):
    """Slices (b0, b1, h0, h1) per rank.  Batch first; heads are split only when the batch alone
    cannot give every rank the same amount of work."""
    if world <= 0:
        raise ValueError("world must be positive")
    if b % world == 0:
        per = b // world
        return [(r * per, (r + 1) * per, 0, h) for r in range(world)]
    if world % b == 0 and h % (world // b) == 0:
        split = world // b
        hp = h // split
        return [(r // split, r // split + 1, (r % split) * hp, (r % split + 1) * hp) for r in range(world)]
    per = -(-b // world)
    return [(min(r * per, b), min((r + 1) * per, b), 0, h) for r in range(world)]


def shard_rows(x, a, rank, world):
    """This rank's views of x[b,L,h,d] and a[b,L,h] | a[h] (no copies)."""
    b0, b1, h0, h1 = plan_row_shards(x.shape[0], x.shape[2], world)[rank]
    xs = x[b0:b1, :, h0:h1]
    a_s = a[h0:h1] if a.dim() == 1 else a[b0:b1, :, h0:h1]
    return xs, a_s


class _RowShardedEma(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, a, group, backend, heads_replicated):
        r = backend.ema_fwd(x, a, want_tile_states=True)
        ctx.save_for_backward(x, a, r["tile_states"])
        ctx.group, ctx.backend, ctx.heads_replicated = group, backend, heads_replicated
        return r["y"]

    @staticmethod
    def backward(ctx, dy):
        x, a, ts = ctx.saved_tensors
        r = ctx.backend.ema_bwd(x, a, dy, ts)
        da = r["ddecay"]
        if a.dim() == 1 and ctx.heads_replicated:
            dist.all_reduce(da, group=ctx.group)  # the only collective: h floats
        return r["dx"], da, None, None, None


def ema_row_sharded(x_local, a_local, group=None, backend=None, heads_replicated=True):
    """EMA of this rank's row shard.  `heads_replicated` says that the same heads (hence the same
    a[h]) live on several ranks, i.e. the batch was what got sharded."""
    return _RowShardedEma.apply(x_local, a_local, group, backend or _cuda_ops, heads_replicated)


# ---- sequence parallel ------------------------------------------------------------------------

def fold_carries(finals, log_sums, upto):
    """State entering segment `upto` given zero-state finals F_j and summed log-decays of segments
    0..upto-1:  carry <- exp(logP_j) carry + F_j."""
    carry = torch.zeros_like(finals[0])
    for j in range(upto):
        carry = torch.exp(log_sums[j]).unsqueeze(-1) * carry + finals[j]
    return carry


def fold_adjoints(dinits, log_sums, after):
    """Adjoint entering segment `after` from the right, given the zero-carry dinit G_j of segments
    after+1..W-1:  carry <- exp(logP_j) carry + G_j, right to left."""
    carry = torch.zeros_like(dinits[0])
    for j in range(len(dinits) - 1, after, -1):
        carry = torch.exp(log_sums[j]).unsqueeze(-1) * carry + dinits[j]
    return carry


def _gather_records(rec, group):
    """[world, n] from every rank's flat record [n] (one collective)."""
    world = dist.get_world_size(group)
    out = torch.empty((world * rec.numel(),), dtype=rec.dtype, device=rec.device)
    dist.all_gather_into_tensor(out, rec, group=group)
    return out.view(world, rec.numel())


def _fold(backend, records, rank, b, h, d, reverse):
    """Folds the gathered records [world, b*h*d + b*h] into the carry entering segment `rank`: one kernel when the
    backend has one (CUDA), otherwise the torch loops above (the CPU stand-in of the tests)."""
    rows = b * h
    if hasattr(backend, "fold_records"):
        return backend.fold_records(records, rank, rows, d, reverse=reverse).view(b, h, d)
    vecs = [r[:rows * d].view(b, h, d) for r in records]
    logs = [r[rows * d:].view(b, h) for r in records]
    return fold_adjoints(vecs, logs, rank) if reverse else fold_carries(vecs, logs, rank)


class _SeqParallelEma(torch.autograd.Function):
    """Local scan from a zero state, ONE all-gather of [final state | summed log decay] per direction, fold, and a
    re-scan of the part of the segment the incoming carry can still change."""

    @staticmethod
    def forward(ctx, x, a, group, backend, stop_below):
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        b, L, h, d = x.shape
        rows = b * h
        # the record this rank contributes: the kernel writes both parts straight into it
        rec = torch.empty((rows * d + rows,), dtype=torch.float32, device=x.device)
        fin, lds = rec[:rows * d].view(b, h, d), rec[rows * d:].view(b, h)
        _mark("fwd_begin", x)
        r = backend.ema_fwd(x, a, want_tile_states=True, want_final=True, want_log_decay_sum=True, final_out=fin,
                            log_decay_sum_out=lds)
        if r["final_state"].data_ptr() != fin.data_ptr():   # a backend that allocates its own outputs
            fin.copy_(r["final_state"])
            lds.copy_(r["log_decay_sum"])
        y, ts = r["y"], r["tile_states"]
        _mark("fwd_local", x)
        if world > 1:
            records = _gather_records(rec, group)
            carry_in = _fold(backend, records, rank, b, h, d, reverse=False) if rank > 0 else None
            _mark("fwd_exchange", x)
            if rank > 0:
                backend.ema_fwd(x, a, init_state=carry_in, stop_below=stop_below, out=y, tile_states=ts)
        _mark("fwd_end", x)
        ctx.save_for_backward(x, a, ts, lds)
        ctx.group, ctx.backend, ctx.stop_below = group, backend, stop_below
        ctx.rank, ctx.world = rank, world
        return y

    @staticmethod
    def backward(ctx, dy):
        x, a, ts, lds = ctx.saved_tensors
        backend, group = ctx.backend, ctx.group
        b, L, h, d = x.shape
        rows = b * h
        rec = torch.empty((rows * d + rows,), dtype=torch.float32, device=x.device)
        dinit = rec[:rows * d].view(b, h, d)
        rec[rows * d:].copy_(lds.reshape(-1))
        _mark("bwd_begin", x)
        r = backend.ema_bwd(x, a, dy, ts, want_dinit=True, dinit_out=dinit)
        if r["dinit_state"].data_ptr() != dinit.data_ptr():
            dinit.copy_(r["dinit_state"])
        _mark("bwd_local", x)
        if ctx.world > 1:
            records = _gather_records(rec, group)
            last = ctx.rank == ctx.world - 1
            dfinal = None if last else _fold(backend, records, ctx.rank, b, h, d, reverse=True)
            _mark("bwd_exchange", x)
            if not last:
                r = backend.ema_bwd(x, a, dy, ts, dfinal_state=dfinal, stop_below=ctx.stop_below, dx=r["dx"],
                                    workspace=r["workspace"], ddecay=r["ddecay"])
        da = r["ddecay"]
        if a.dim() == 1 and ctx.world > 1:
            dist.all_reduce(da, group=group)
        _mark("bwd_end", x)
        return r["dx"], da, None, None, None


def ema_sequence_parallel(x_seg, a_seg, group=None, backend=None, stop_below=STOP_BELOW):
    """EMA over a sequence split into contiguous per-rank segments (rank order = sequence order).
    x_seg[b, L/W, h, d], a_seg[b, L/W, h] or a[h]; differentiable."""
    return _SeqParallelEma.apply(x_seg, a_seg, group, backend or _cuda_ops, stop_below)
