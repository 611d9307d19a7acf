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
chunked kernels) is a decay of exactly 0 at the first step of every new sequence.  State sizes above 1 and
cu_seqlens (variable-length final states) are rejected: they belong to the general state-space scan.
"""
import torch
import torch.nn.functional as F

from ema_b200 import ops


class _WeightedScan(torch.autograd.Function):
    """y_t = c_t s_t, s_t = exp(A_t) s_{t-1} + w_t x_t over x[b,L,h,p] with per-step A, w, c [b,L,h] (fp32) and an
    optional initial state: forward and backward are one kernel pass each, the weights folded into the scan, and the
    gradients of A, w, c come out of the backward pass as [b,L,h] tensors."""

    @staticmethod
    def forward(ctx, x, a_log, w, c, init_state):
        r = ops.ema_fwd(x, a_log, prescaled_log=True, init_state=init_state, want_tile_states=True, want_final=True,
                        in_weight=w, out_weight=c)
        ctx.save_for_backward(x, a_log, w, c, r["tile_states"])
        ctx.has_init = init_state is not None
        return r["y"], r["final_state"]

    @staticmethod
    def backward(ctx, dy, dfinal):
        x, a_log, w, c, tile_states = ctx.saved_tensors
        r = ops.ema_bwd_weighted(x, a_log, dy.contiguous(), tile_states, in_weight=w, out_weight=c, prescaled_log=True,
                                 dfinal_state=None if dfinal is None else dfinal.float().contiguous(),
                                 want_dinit=ctx.has_init)
        return r["dx"], r["ddecay"], r["din_weight"], r["dout_weight"], r.get("dinit_state")


def _processed_dt(dt, dt_bias, dt_softplus, dt_limit):
    dt = dt.float()
    if dt_bias is not None:
        dt = dt + dt_bias.float()
    if dt_softplus:
        dt = torch.where(dt <= 20.0, F.softplus(dt), dt)
    return torch.clamp(dt, min=dt_limit[0], max=dt_limit[1])


def _ema_chunk_scan_combined_fwd(x, dt, A, B, C, chunk_size, D=None, z=None, dt_bias=None, initial_states=None,
                                 seq_idx=None, cu_seqlens=None, dt_softplus=False, dt_limit=(0.0, float("inf"))):
    """Same checks and same role as the reference's function of this name (:12-66); returns (out, final_states).
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
    if cu_seqlens is not None:
        raise NotImplementedError("cu_seqlens (variable-length final states) is not part of the EMA path")
    if seq_idx is not None:
        assert seq_idx.shape == (batch, seqlen)
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
    if not needs_grad and D is None and z is None:
        # inference: the weights dt' B (input) and C (output) go into the scan kernel itself, so x is read once and the
        # result written once; only the [b, l, h]-sized weight tensors are prepared here
        r = ops.ema_fwd(x, a_log.contiguous(), prescaled_log=True, init_state=init, want_final=True,
                        in_weight=(dtp * Bh).contiguous(), out_weight=Ch.contiguous())
        return r["y"], r["final_state"].unsqueeze(-1)
    # training: the same folding, with the gradients of the decay and of both weights returned by the backward pass as
    # [b, l, h] tensors; autograd carries them on to dt, A, B, C, dt_bias (small elementwise work)
    s, final = _WeightedScan.apply(x.contiguous() if x.stride(-1) != 1 else x, a_log.contiguous(),
                                   (dtp * Bh).contiguous(), Ch.contiguous(), init)
    if D is None and z is None:
        return s, final.unsqueeze(-1)
    out = s.float()
    if D is not None:
        out = out + x.float() * (D.float().unsqueeze(-1) if D.dim() == 1 else D.float())
    if z is not None:
        out = out * F.silu(z.float())
    return out.to(x.dtype), final.unsqueeze(-1)


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
    Return:
        out: (batch, seqlen, nheads, headdim), and final_states (batch, nheads, headdim, 1) if asked for
    """
    if return_varlen_states:
        raise NotImplementedError("varlen states are not part of the EMA path")
    out, final = _ema_chunk_scan_combined_fwd(x, dt, A, B, C, chunk_size, D=D, z=z, dt_bias=dt_bias,
                                              initial_states=initial_states, seq_idx=seq_idx, cu_seqlens=cu_seqlens,
                                              dt_softplus=dt_softplus, dt_limit=dt_limit)
    return (out, final) if return_final_states else out
