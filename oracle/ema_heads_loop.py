"""Sequential fp64 definition of the reference's heads-style entry point for state size 1.  TEST INFRASTRUCTURE ONLY.

Follows ema_chunk_scan_combined of the reference (kernels/ema_combined.py:100, forward :12-57):

    dt'  = clamp(softplus?(dt + dt_bias), dt_limit)                        kernels/ema_chunk_state.py:69-78
    s_t  = exp(dt'_t A_h) s_{t-1} + dt'_t B_t x_t                           (state restarts from zero where seq_idx changes)
    y_t  = C_t s_t  (+ D x_t)  (* silu(z_t))

The reference's cumulative-sum kernel hard-codes the log decay as -dt' (kernels/ema_chunk_state.py:95), i.e. it
ignores A; the loop below uses A, and is pinned against fixtures recorded from the reference with A = -1
(tests/golden/heads_*.npz, tests/test_oracle.py).  numpy for values, a torch twin for gradients by autograd.
"""
import numpy as np


def _softplus(v):
    return np.where(v <= 20.0, np.log1p(np.exp(np.minimum(v, 20.0))), v)


def processed_dt(dt, dt_bias=None, dt_softplus=False, dt_limit=(0.0, float("inf"))):
    d = dt.astype(np.float64)
    if dt_bias is not None:
        d = d + dt_bias.astype(np.float64)
    if dt_softplus:
        d = _softplus(d)
    return np.clip(d, dt_limit[0], dt_limit[1])


def heads_loop(x, dt, A, B, C, D=None, z=None, dt_bias=None, initial_states=None, dt_softplus=False,
               dt_limit=(0.0, float("inf")), seq_idx=None, cu_seqlens=None, chunk_size=None):
    """x[b,L,h,p], dt[b,L,h], A[h], B/C[b,L,g,1] -> (out[b,L,h,p], final_states[b,h,p,1]) in float64.
    With cu_seqlens (batch 1, packed sequences; seq_idx must mark the same boundaries) a third value: the state after
    the last step of every sequence, [num_sequences, h, p, 1] (return_varlen_states of the reference,
    kernels/ema_combined.py:56-62).  The reference adds the state entering the chunk that holds a sequence's end only
    when the sequence starts before that chunk (kernels/ema_chunk_state.py:560-566): a first sequence that ends inside
    the first chunk therefore comes out WITHOUT initial_states, and so it does here (chunk_size must then be given)."""
    b, L, h, p = x.shape
    rep = h // B.shape[2]
    d = processed_dt(dt, dt_bias, dt_softplus, dt_limit)
    Bh = np.repeat(B[..., 0].astype(np.float64), rep, axis=2)
    Ch = np.repeat(C[..., 0].astype(np.float64), rep, axis=2)
    xs = x.astype(np.float64)
    s = np.zeros((b, h, p)) if initial_states is None else initial_states[..., 0].astype(np.float64).copy()
    out = np.empty((b, L, h, p))
    ends = {} if cu_seqlens is None else {int(e) - 1: i for i, e in enumerate(np.asarray(cu_seqlens)[1:])}
    varlen = np.zeros((len(ends), h, p))
    s_init = s.copy()   # what is left of initial_states alone
    for t in range(L):
        if seq_idx is not None and t > 0:
            same = (seq_idx[:, t] == seq_idx[:, t - 1]).astype(np.float64).reshape(b, 1, 1)
            s, s_init = s * same, s_init * same
        a_t = np.exp(d[:, t] * A.astype(np.float64))[..., None]
        s = a_t * s + (d[:, t] * Bh[:, t])[..., None] * xs[:, t]
        s_init = a_t * s_init
        out[:, t] = Ch[:, t][..., None] * s
        if t in ends:
            varlen[ends[t]] = s[0]
            if ends[t] == 0 and initial_states is not None and t // chunk_size == 0:
                varlen[0] -= s_init[0]
    if D is not None:
        Dd = D.astype(np.float64)
        out = out + xs * (Dd[:, None] if Dd.ndim == 1 else Dd)
    if z is not None:
        zz = z.astype(np.float64)
        out = out * (zz / (1.0 + np.exp(-zz)))
    if cu_seqlens is not None:
        assert b == 1
        return out, s[..., None], varlen[..., None]
    return out, s[..., None]


def heads_loop_torch(x, dt, A, B, C, D=None, z=None, dt_bias=None, initial_states=None, dt_softplus=False,
                     dt_limit=(0.0, float("inf")), seq_idx=None):
    """The same loop on torch tensors (any dtype, normally float64 leaves), differentiable by autograd."""
    import torch
    import torch.nn.functional as F
    b, L, h, p = x.shape
    rep = h // B.shape[2]
    d = dt if dt_bias is None else dt + dt_bias
    if dt_softplus:
        d = torch.where(d <= 20.0, F.softplus(d), d)
    d = torch.clamp(d, min=dt_limit[0], max=dt_limit[1])
    Bh = B[..., 0].repeat_interleave(rep, dim=2)
    Ch = C[..., 0].repeat_interleave(rep, dim=2)
    s = torch.zeros((b, h, p), dtype=x.dtype) if initial_states is None else initial_states[..., 0]
    ys = []
    for t in range(L):
        if seq_idx is not None and t > 0:
            s = s * (seq_idx[:, t] == seq_idx[:, t - 1]).to(s.dtype).view(b, 1, 1)
        s = torch.exp(d[:, t] * A).unsqueeze(-1) * s + (d[:, t] * Bh[:, t]).unsqueeze(-1) * x[:, t]
        ys.append(Ch[:, t].unsqueeze(-1) * s)
    y = torch.stack(ys, dim=1)
    if D is not None:
        y = y + x * (D.unsqueeze(-1) if D.dim() == 1 else D)
    if z is not None:
        y = y * F.silu(z)
    return y, s.unsqueeze(-1)
