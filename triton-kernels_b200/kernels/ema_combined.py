"""Drop-in for kernels/ema_combined.py of the reference: the heads-style entry point

    ema_chunk_scan_combined(x[b,l,h,p], dt[b,l,h], A[h], B[b,l,g,n], C[b,l,g,n], chunk_size, ...)   (:100)

for the EMA special case, state size n = 1 (the only case the reference's EMA callers use: B = the input
weight, C = 1, kernels/benchmarks/ema_bench.py:104-117):

    dt'  = clamp(softplus?(dt + dt_bias), dt_limit)                      (ema_chunk_state.py:69-78)
    s_t  = exp(dt'_t A_h) s_{t-1} + dt'_t B_t x_t ,     y_t = C_t s_t  (+ D x_t)  (* silu(z_t))

The recurrence runs in the fused scan kernels (pre-scaled log-decay convention: decay = dt' A) with the weights dt' B
(input) and C (output) folded into the kernels: one read of x and one write of the result forward, one read of x and
dy and one write of dx backward.  The backward pass also returns the gradients of the decay and of both weights as
[b, l, h] tensors, from which autograd reaches dt, A, B, C and dt_bias on [b, l, h]-sized data.  Only D and z, when
given, add elementwise torch work on the full-size tensors.
The reference's own backward for this entry point is a stub that returns None for every input (:89-92).
`seq_idx` (a sequence id per position: the state restarts from zero where the id changes, as in the reference's
chunked kernels) is a decay of exactly 0 at the first step of every new sequence.
`cu_seqlens` with `return_varlen_states` (batch 1, packed sequences, :56-62 and ema_chunk_state.py:578): the state after
the last step of every sequence, from the states the scan kernel saves at the chunk boundaries plus the at most
chunk_size steps between the boundary and the sequence's end (a small torch computation per sequence); forward only, as
in the reference.  State sizes above 1 are rejected: they belong to the general state-space scan.
"""
import torch
import torch.nn.functional as F

from ema_b200 import ops


class _WeightedScan(torch.autograd.Function):
    """y_t = c_t s_t, s_t = exp(A_t) s_{t-1} + w_t x_t over x[b,L,h,p] with per-step A, w, c [b,L,h] (fp32) and an
    optional initial state: forward and backward are one kernel pass each, the weights folded into the scan, and the
    gradients of A, w, c come out of the backward pass as [b,L,h] tensors."""

    @staticmethod
    def forward(ctx, x, a_log, w, c, init_state, chunk=0):
        r = ops.ema_fwd(x, a_log, prescaled_log=True, init_state=init_state, want_tile_states=True, want_final=True,
                        in_weight=w, out_weight=c, chunk=chunk, want_chunk_states=chunk > 0)
        ctx.save_for_backward(x, a_log, w, c, r["tile_states"])
        ctx.has_init = init_state is not None
        ctx.has_chunks = chunk > 0
        if chunk > 0:   # states at the chunk boundaries, for the variable-length states (not differentiable)
            ctx.mark_non_differentiable(r["chunk_states"])
            return r["y"], r["final_state"], r["chunk_states"]
        return r["y"], r["final_state"]

    @staticmethod
    def backward(ctx, dy, dfinal, *unused):
        assert not ctx.has_chunks, "return_varlen_states is not supported in backward"
        x, a_log, w, c, tile_states = ctx.saved_tensors
        r = ops.ema_bwd_weighted(x, a_log, dy.contiguous(), tile_states, in_weight=w, out_weight=c, prescaled_log=True,
                                 dfinal_state=None if dfinal is None else dfinal.float().contiguous(),
                                 want_dinit=ctx.has_init)
        return r["dx"], r["ddecay"], r["din_weight"], r["dout_weight"], r.get("dinit_state"), None


def _processed_dt(dt, dt_bias, dt_softplus, dt_limit):
    dt = dt.float()
    if dt_bias is not None:
        dt = dt + dt_bias.float()
    if dt_softplus:
        dt = torch.where(dt <= 20.0, F.softplus(dt), dt)
    return torch.clamp(dt, min=dt_limit[0], max=dt_limit[1])


def _ema_chunk_scan_combined_fwd(x, dt, A, B, C, chunk_size, D=None, z=None, dt_bias=None, initial_states=None,
                                 seq_idx=None, cu_seqlens=None, dt_softplus=False, dt_limit=(0.0, float("inf"))):
    """Same checks and same role as the reference's function of this name (:12-66); returns (out, final_states), and
    the variable-length states as a third value when cu_seqlens is given.
    (The reference also returns its chunked intermediates; the fused kernels have none to return.)"""
    batch, seqlen, nheads, headdim = x.shape
    _, _, ngroups, dstate = B.shape
    assert nheads % ngroups == 0
    assert B.shape == (batch, seqlen, ngroups, dstate)
    assert dt.shape == (batch, seqlen, nheads)
    assert A.shape == (nheads,)
    assert C.shape == B.shape
    if z is not None:
        assert z.shape == x.shape
    if D is not None:
        assert D.shape == (nheads, headdim) or D.shape == (nheads,)
    if dstate != 1:
        raise NotImplementedError("only the EMA special case (state size 1) is built on this path")
    if seq_idx is not None:
        assert seq_idx.shape == (batch, seqlen)
    chunk = 0
    if cu_seqlens is not None:
        assert batch == 1, "passing cu_seqlens to get the varlen states is only supported if batch dimension is 1"
        cu = [int(v) for v in cu_seqlens.tolist()]
        starts = torch.zeros(seqlen, dtype=torch.bool, device=x.device)
        if len(cu) > 2:
            starts[torch.tensor(cu[1:-1], device=x.device)] = True
        marked = torch.zeros_like(starts)
        if seq_idx is not None:
            marked[1:] = seq_idx[0, 1:] != seq_idx[0, :-1]
        if cu[0] != 0 or cu[-1] != seqlen or not torch.equal(starts, marked):
            # without restarts at the same places the reference's states depend on where its chunks happen to fall
            raise NotImplementedError("cu_seqlens needs a seq_idx that changes exactly at cu_seqlens[1:-1]")
        chunk = int(chunk_size)
    if initial_states is not None:
        assert initial_states.shape == (batch, nheads, headdim, dstate)
    rep = nheads // ngroups
    dtp = _processed_dt(dt, dt_bias, dt_softplus, dt_limit)                     # [b, l, h] fp32
    a_log = dtp * A.float()                                                      # log decay per step
    if seq_idx is not None:   # a new sequence starts from a zero state: log decay -inf, i.e. decay 0, at its first step
        new_seq = torch.zeros_like(seq_idx, dtype=torch.bool)
        new_seq[:, 1:] = seq_idx[:, 1:] != seq_idx[:, :-1]
        a_log = a_log.masked_fill(new_seq.unsqueeze(-1), float("-inf"))
    Bh = B[..., 0].float().repeat_interleave(rep, dim=2)                         # [b, l, h]
    Ch = C[..., 0].float().repeat_interleave(rep, dim=2)
    init = None if initial_states is None else initial_states[..., 0].float().contiguous()
    needs_grad = torch.is_grad_enabled() and any(
        t is not None and t.requires_grad for t in (x, dt, A, B, C, D, z, dt_bias, initial_states))
    w_in = (dtp * Bh).contiguous()

    def with_varlen(out, final, chunk_states):
        if cu_seqlens is None:
            return out, final
        return out, final, _varlen_states(x, a_log, w_in, chunk_states, cu, chunk)

    if not needs_grad and D is None and z is None:
        # inference: the weights dt' B (input) and C (output) go into the scan kernel itself, so x is read once and the
        # result written once; only the [b, l, h]-sized weight tensors are prepared here
        r = ops.ema_fwd(x, a_log.contiguous(), prescaled_log=True, init_state=init, want_final=True,
                        in_weight=w_in, out_weight=Ch.contiguous(), chunk=chunk, want_chunk_states=chunk > 0)
        return with_varlen(r["y"], r["final_state"].unsqueeze(-1), r.get("chunk_states"))
    # training: the same folding, with the gradients of the decay and of both weights returned by the backward pass as
    # [b, l, h] tensors; autograd carries them on to dt, A, B, C, dt_bias (small elementwise work)
    res = _WeightedScan.apply(x.contiguous() if x.stride(-1) != 1 else x, a_log.contiguous(), w_in, Ch.contiguous(), init,
                              chunk)
    s, final, chunk_states = res[0], res[1], (res[2] if chunk > 0 else None)
    if D is None and z is None:
        return with_varlen(s, final.unsqueeze(-1), chunk_states)
    out = s.float()
    if D is not None:
        out = out + x.float() * (D.float().unsqueeze(-1) if D.dim() == 1 else D.float())
    if z is not None:
        out = out * F.silu(z.float())
    return with_varlen(out.to(x.dtype), final.unsqueeze(-1), chunk_states)


def _varlen_states(x, a_log, w_in, chunk_states, cu, chunk):
    """State after the last step of every packed sequence (batch 1), [num_sequences, h, p, 1] fp32: the state the scan
    kernel saved at the start of the chunk that holds the sequence's end, carried over the steps from there to the end.
    As in the reference (kernels/ema_chunk_state.py:560-566) the saved state counts only when the sequence starts before
    that chunk; a sequence that starts inside it has restarted from zero anyway - except the very first one, whose
    initial_states the reference thereby leaves out when it ends inside the first chunk, and so does this."""
    h, p = x.shape[2], x.shape[3]
    out = torch.empty((len(cu) - 1, h, p), dtype=torch.float32, device=x.device)
    saved = chunk_states.view(h, -1, p)               # [scan rows = heads (batch 1), chunks, channels]
    for i in range(len(cu) - 1):
        start, end = cu[i], cu[i + 1]
        if end <= start:
            out[i] = 0.0
            continue
        t0 = ((end - 1) // chunk) * chunk
        lw = a_log[0, t0:end].float()                                              # [n, h] log decays, -inf at a restart
        after = torch.flip(torch.cumsum(torch.flip(lw, [0]), 0), [0])                # sum over steps t .. end-1
        factor = torch.exp(torch.cat([after[1:], torch.zeros_like(after[:1])], 0))   # decay from step t to the end
        wx = w_in[0, t0:end].unsqueeze(-1) * x[0, t0:end].float()                   # [n, h, p]
        s = (factor.unsqueeze(-1) * wx).sum(0)
        if start < t0:
            s = s + torch.exp(after[0]).unsqueeze(-1) * saved[:, t0 // chunk]
        out[i] = s
    return out.unsqueeze(-1)


def ema_chunk_scan_combined(x, dt, A, B, C, chunk_size, D=None, z=None, dt_bias=None, initial_states=None,
                            seq_idx=None, cu_seqlens=None, dt_softplus=False, dt_limit=(0.0, float("inf")),
                            return_final_states=False, return_varlen_states=False):
    """
    Argument:
        x: (batch, seqlen, nheads, headdim)
        dt: (batch, seqlen, nheads)
        A: (nheads)
        B, C: (batch, seqlen, ngroups, 1)
        chunk_size: int (accepted for compatibility; the kernels choose their own tile)
        D: (nheads, headdim) or (nheads,)
        z: (batch, seqlen, nheads, headdim)
        dt_bias: (nheads,)
        initial_states: (batch, nheads, headdim, 1)
        dt_softplus: whether to apply softplus to dt
        seq_idx: (batch, seqlen)
        cu_seqlens: (num_sequences + 1) or None, only used if return_varlen_states is True
    Return:
        out: (batch, seqlen, nheads, headdim); then final_states (batch, nheads, headdim, 1) if return_final_states;
        then varlen_states (num_sequences, nheads, headdim, 1) if return_varlen_states
    """
    if not return_varlen_states:
        cu_seqlens = None
    else:
        assert cu_seqlens is not None, "cu_seqlens must be provided if return_varlen_states is True"
    res = _ema_chunk_scan_combined_fwd(x, dt, A, B, C, chunk_size, D=D, z=z, dt_bias=dt_bias,
                                       initial_states=initial_states, seq_idx=seq_idx, cu_seqlens=cu_seqlens,
                                       dt_softplus=dt_softplus, dt_limit=dt_limit)
    out, final = res[0], res[1]
    if not return_varlen_states:
        return (out, final) if return_final_states else out
    return (out, final, res[2]) if return_final_states else (out, res[2])
