"""numpy restatement of every stage of the reference's chunked EMA pipeline.  TEST INFRASTRUCTURE ONLY.

Each function follows one reference stage (file:line given per function) on the reference's own
layouts: X[B,L,T] (pre-scaled input u), A[B,L] (log-decay), cs[B,C,Q], states [B,C,T].
Computation is float64 inside, float32 out.  Pinned by tests/test_oracle.py against the outputs
of the reference's Triton kernels run under Triton's interpreter (tests/golden/stages_*.npz).
"""
import math

import numpy as np


def _chunks(L, Q):
    return math.ceil(L / Q)


def _pad_time(v, Q):
    """[B,L,...] -> [B,C,Q,...] zero padded."""
    B, L = v.shape[:2]
    C = _chunks(L, Q)
    out = np.zeros((B, C * Q) + v.shape[2:], np.float64)
    out[:, :L] = v
    return out.reshape((B, C, Q) + v.shape[2:])


def chunk_cumsum(A, Q):
    """kernels/ema_kernels/ema_cumsum.py:32-63: per-chunk inclusive cumsum, tail zero padded."""
    return np.cumsum(_pad_time(A, Q), axis=2).astype(np.float32)


def _limits(L, Q):
    C = _chunks(L, Q)
    return np.minimum(Q, L - np.arange(C) * Q)


def chunk_state(X, cs):
    """kernels/ema_kernels/ema_state_fwd.py:98-122: S_c = sum_q exp(min(cs_last - cs_q, 0)) u_q,
    cs_last read at the last VALID position of the chunk."""
    B, L, T = X.shape
    _, C, Q = cs.shape
    lim = _limits(L, Q)
    cs64 = cs.astype(np.float64)
    last = cs64[:, np.arange(C), lim - 1]
    w = np.exp(np.minimum(last[:, :, None] - cs64, 0.0))
    return np.einsum("bcq,bcqt->bct", w, _pad_time(X, Q)).astype(np.float32)


def state_passing_fwd(S, cs_last):
    """kernels/ema_kernels/ema_state_pass.py:100-120: out[c] = state at the start of chunk c."""
    B, C, T = S.shape
    out = np.zeros((B, C, T), np.float64)
    acc = np.zeros((B, T), np.float64)
    for c in range(C):
        out[:, c] = acc
        acc = np.exp(cs_last[:, c].astype(np.float64))[:, None] * acc + S[:, c]
    return out.astype(np.float32), acc.astype(np.float32)


def chunk_scan(X, cs, h):
    """kernels/ema_kernels/ema_scan_fwd.py:111-156:
    y_m = exp(min(cs_m,0)) h_c + sum_{k<=m} exp(min(cs_m - cs_k,0)) u_k."""
    B, L, T = X.shape
    _, C, Q = cs.shape
    cs64 = cs.astype(np.float64)
    Lmat = np.exp(np.minimum(cs64[:, :, :, None] - cs64[:, :, None, :], 0.0)) * np.tril(np.ones((Q, Q)))
    y = np.einsum("bcmk,bckt->bcmt", Lmat, _pad_time(X, Q))
    y += np.exp(np.minimum(cs64, 0.0))[..., None] * h.astype(np.float64)[:, :, None, :]
    return y.reshape(B, C * Q, T)[:, :L].astype(np.float32)


def bwd_dstates(cs, dout):
    """kernels/ema_kernels_bwd/ema_scan_bwd.py:96-110: dh_scan[c] = sum_q exp(cs_q) dy_q."""
    _, C, Q = cs.shape
    return np.einsum("bcq,bcqt->bct", np.exp(cs.astype(np.float64)), _pad_time(dout, Q)).astype(np.float32)


def state_passing_bwd(h, cs_last, dh_scan):
    """kernels/ema_kernels_bwd/ema_state_passing_bwd_dstates.py:60-98: reverse carry of the adjoint.
    dS[c] = adjoint of chunk c's local state; ddA_last[c] = exp(cs_last_c) <h_c, dS[c]>, forced to 0
    for chunk 0."""
    B, C, T = h.shape
    dS = np.zeros((B, C, T), np.float64)
    ddA = np.zeros((B, C), np.float64)
    g = np.zeros((B, T), np.float64)
    for c in range(C - 1, 0, -1):
        dS[:, c] = g
        scale = np.exp(cs_last[:, c].astype(np.float64))
        ddA[:, c] = (h[:, c].astype(np.float64) * g).sum(-1) * scale
        g = scale[:, None] * g + dh_scan[:, c]
    dS[:, 0] = g
    return dS.astype(np.float32), ddA.astype(np.float32)


def bwd_dx(cs, dout, dS, L):
    """kernels/ema_kernels_bwd/ema_chunk_scan_chunk_state_bwd_dx.py:126-189:
    du_m = exp(min(cs_last - cs_m,0)) dS_c + sum_{k>=m} exp(min(cs_k - cs_m,0)) dy_k."""
    B, C, Q = cs.shape
    T = dout.shape[-1]
    cs64 = cs.astype(np.float64)
    W = np.exp(np.minimum(cs64[:, :, None, :] - cs64[:, :, :, None], 0.0)) * np.triu(np.ones((Q, Q)))
    du = np.einsum("bcmk,bckt->bcmt", W, _pad_time(dout, Q))
    du += np.exp(np.minimum(cs64[:, :, -1:] - cs64, 0.0))[..., None] * dS.astype(np.float64)[:, :, None, :]
    return du.reshape(B, C * Q, T)[:, :L].astype(np.float32)


def bwd_db(X, cs, dS, raw=False):
    """kernels/ema_kernels_bwd/ema_chunk_state_bwd_db.py:75-117,151: g_m = exp(min(cs_last-cs_m,0))
    <dS_c,u_m> stored at slot m+1 (valid m < limit-1), then cumsum along the chunk unless raw."""
    B, L, T = X.shape
    _, C, Q = cs.shape
    lim = _limits(L, Q)
    cs64 = cs.astype(np.float64)
    g = np.einsum("bct,bcqt->bcq", dS.astype(np.float64), _pad_time(X, Q))
    g *= np.exp(np.minimum(cs64[:, :, -1:] - cs64, 0.0))
    out = np.zeros((B, C, Q), np.float64)
    for c in range(C):
        n = lim[c] - 1
        out[:, c, 1:n + 1] = g[:, c, :n]
    return (out if raw else np.cumsum(out, axis=-1)).astype(np.float32)


def bwd_dc(h, cs, dout):
    """kernels/ema_kernels_bwd/ema_chunk_scan_bwd_dc.py:82-112: r_m = exp(cs_m) <dy_m, h_c>,
    zero past the end of a ragged last chunk."""
    _, C, Q = cs.shape
    r = np.einsum("bcqt,bct->bcq", _pad_time(dout, Q), h.astype(np.float64))
    return (r * np.exp(cs.astype(np.float64))).astype(np.float32)


def bwd_dacs(X, cs, dout):
    """kernels/ema_kernels_bwd/ema_scan_da.py:69-106,136: G[m,k] = <dy_m,u_k> exp(min(cs_m-cs_k,0))
    for m>k; out[j+1] = sum_{m>j} sum_{k<=j} G[m,k]; out[0] = 0."""
    B, C, Q = cs.shape
    cs64 = cs.astype(np.float64)
    G = np.einsum("bcmt,bckt->bcmk", _pad_time(dout, Q), _pad_time(X, Q))
    G *= np.exp(np.minimum(cs64[:, :, :, None] - cs64[:, :, None, :], 0.0)) * np.tril(np.ones((Q, Q)), -1)
    Gc = np.cumsum(G, axis=-1)                      # sum over k <= j
    out = np.zeros((B, C, Q), np.float64)
    for j in range(Q - 1):
        out[:, :, j + 1] = Gc[:, :, j + 1:, j].sum(axis=-1)
    return out.astype(np.float32)


def combined_bwd(dout, X, A, Q):
    """kernels/ema_kernels_bwd/ema_combined_bwd.py:13-82: (dx, ddA[B,C,Q])."""
    B, L, T = X.shape
    cs = chunk_cumsum(A, Q)
    S = chunk_state(X, cs)
    h, _ = state_passing_fwd(S, cs[..., -1])
    dh = bwd_dstates(cs, dout)
    dS, ddA_last = state_passing_bwd(h, cs[..., -1], dh)
    dx = bwd_dx(cs, dout, dS, L)
    nxt = bwd_db(X, cs, dS).astype(np.float64)
    prev = bwd_dc(h, cs, dout).astype(np.float64)
    prev[..., -1] += ddA_last
    prev = np.cumsum(prev[..., ::-1], axis=-1)[..., ::-1]
    return dx, (bwd_dacs(X, cs, dout) + nxt + prev).astype(np.float32)
