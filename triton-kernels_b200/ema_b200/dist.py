"""Multi-GPU EMA: one process per GPU, torch.distributed (NCCL over NVLink) for the plumbing.

Two modes, neither of which exists in the reference project (it is single-GPU):

* row sharding - the scan rows (b, h) are independent, so every rank scans its own slice with no
  data-path collective.  Only a time-invariant decay a[h] needs one all-reduce of h floats for its
  gradient.
* sequence parallel - rank g holds the g-th contiguous segment of the sequence.  Every rank scans
  its segment from a zero state, the ranks all-gather the per-row final state F[b,h,d] and the
  summed log-decay logP[b,h] (kept in the log domain: the product of 65536 decays underflows), each
  rank folds its predecessors into its incoming carry, and a fix-up pass re-scans only the prefix of
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


def _all_gather(t, group):
    world = dist.get_world_size(group)
    out = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(out, t.contiguous(), group=group)
    return out


class _SeqParallelEma(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, a, group, backend, stop_below):
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        r = backend.ema_fwd(x, a, want_tile_states=True, want_final=True, want_log_decay_sum=True)
        finals = _all_gather(r["final_state"], group)
        log_sums = _all_gather(r["log_decay_sum"], group)
        y, ts = r["y"], r["tile_states"]
        carry_in = None
        if rank > 0:
            carry_in = fold_carries(finals, log_sums, rank)
            backend.ema_fwd(x, a, init_state=carry_in, stop_below=stop_below, out=y, tile_states=ts)
        ctx.save_for_backward(x, a, ts, torch.stack(log_sums))
        ctx.group, ctx.backend, ctx.stop_below = group, backend, stop_below
        ctx.rank, ctx.world = rank, world
        return y

    @staticmethod
    def backward(ctx, dy):
        x, a, ts, log_sums = ctx.saved_tensors
        backend, group = ctx.backend, ctx.group
        r = backend.ema_bwd(x, a, dy, ts, want_dinit=True)
        dinits = _all_gather(r["dinit_state"], group)
        if ctx.rank < ctx.world - 1:
            dfinal = fold_adjoints(dinits, list(log_sums), ctx.rank)
            r = backend.ema_bwd(x, a, dy, ts, dfinal_state=dfinal, stop_below=ctx.stop_below, dx=r["dx"],
                                workspace=r["workspace"], ddecay=r["ddecay"])
        da = r["ddecay"]
        if a.dim() == 1:
            dist.all_reduce(da, group=group)
        return r["dx"], da, None, None, None


def ema_sequence_parallel(x_seg, a_seg, group=None, backend=None, stop_below=STOP_BELOW):
    """EMA over a sequence split into contiguous per-rank segments (rank order = sequence order).
    x_seg[b, L/W, h, d], a_seg[b, L/W, h] or a[h]; differentiable."""
    return _SeqParallelEma.apply(x_seg, a_seg, group, backend or _cuda_ops, stop_below)
