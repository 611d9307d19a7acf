"""Host side of the per-stage kernels, on the reference project's folded layouts.

X, dout: [B, L, T] contiguous (fp32 | bf16);  A: [B, L];  cs: [B, C, Q] fp32;  per-chunk states:
[B, C, T] fp32.  Each function allocates its output like the reference wrapper it stands in for and
makes one C-ABI call on the current stream of the input's device.
"""
import ctypes
import math

import torch

from ._lib import check, dtype_code, lib, ptr, require_cuda, stream_ptr


def _f32c(t):
    return t if (t.dtype == torch.float32 and t.is_contiguous()) else t.float().contiguous()


def _dims(x, cs):
    B, L, T = x.shape
    _, C, Q = cs.shape
    assert cs.shape == (B, math.ceil(L / Q), Q)
    return B, L, T, C, Q


def chunk_cumsum(A, chunk_size):
    assert A.dim() == 2
    dev = require_cuda(A)
    if A.dtype != torch.float32:
        A = A.float()
    B, L = A.shape
    C = math.ceil(L / chunk_size)
    cs = torch.empty(B, C, chunk_size, device=dev, dtype=torch.float32)
    with torch.cuda.device(dev):
        rc = lib().ema_b200_chunk_cumsum(ptr(A), A.stride(0), A.stride(1), ptr(cs), B, L, chunk_size,
                                         stream_ptr(dev))
    check("ema_b200_chunk_cumsum", rc)
    return cs


def chunk_state(x, cs, states=None, states_in_fp32=True):
    dev = require_cuda(x, cs, states)
    B, L, T, C, Q = _dims(x, cs)
    cs = _f32c(cs)
    S = torch.empty(B, C, T, device=dev, dtype=torch.float32)
    with torch.cuda.device(dev):
        rc = lib().ema_b200_chunk_state(ptr(x), ptr(cs), ptr(S), dtype_code(x.dtype), B, L, T, Q, stream_ptr(dev))
    check("ema_b200_chunk_state", rc)
    if states is not None:
        states.copy_(S)
        return states
    return S if states_in_fp32 else S.to(x.dtype)


def state_passing_fwd(states, cs_last, out_dtype=None):
    dev = require_cuda(states, cs_last)
    B, C, T = states.shape
    S = _f32c(states)
    if cs_last.dtype != torch.float32:
        cs_last = cs_last.float()
    out = torch.empty(B, C, T, device=dev, dtype=torch.float32)
    fin = torch.empty(B, T, device=dev, dtype=torch.float32)
    with torch.cuda.device(dev):
        rc = lib().ema_b200_state_passing_fwd(ptr(S), ptr(cs_last), cs_last.stride(0), cs_last.stride(1),
                                              ptr(out), ptr(fin), B, C, T, stream_ptr(dev))
    check("ema_b200_state_passing_fwd", rc)
    out_dtype = states.dtype if out_dtype is None else out_dtype
    return (out if out_dtype == torch.float32 else out.to(out_dtype)), fin


def chunk_scan(x, cs, states):
    dev = require_cuda(x, cs, states)
    B, L, T, C, Q = _dims(x, cs)
    assert states.shape == (B, C, T)
    out = torch.empty(B, L, T, device=dev, dtype=x.dtype)
    with torch.cuda.device(dev):
        rc = lib().ema_b200_chunk_scan(ptr(x), ptr(_f32c(cs)), ptr(_f32c(states)), ptr(out),
                                       dtype_code(x.dtype), B, L, T, Q, stream_ptr(dev))
    check("ema_b200_chunk_scan", rc)
    return out


def bwd_dstates(cs, dout, dtype=None):
    dev = require_cuda(cs, dout)
    B, L, T, C, Q = _dims(dout, cs)
    dh = torch.empty(B, C, T, device=dev, dtype=torch.float32)
    with torch.cuda.device(dev):
        rc = lib().ema_b200_bwd_dstates(ptr(_f32c(cs)), ptr(dout), ptr(dh), dtype_code(dout.dtype), B, L, T, Q,
                                        stream_ptr(dev))
    check("ema_b200_bwd_dstates", rc)
    dtype = cs.dtype if dtype is None else dtype
    return dh if dtype == torch.float32 else dh.to(dtype)


def state_passing_bwd(states, cs_last, dout, dstates_dtype=None):
    dev = require_cuda(states, cs_last, dout)
    B, C, T = states.shape
    if cs_last.dtype != torch.float32:
        cs_last = cs_last.float()
    dS = torch.empty(B, C, T, device=dev, dtype=torch.float32)
    ddA = torch.empty(B, C, device=dev, dtype=torch.float32)
    # partial dot products per 128 channels (the reference's wrapper allocates the same kind of buffer)
    ws_bytes = lib().ema_b200_state_passing_bwd_workspace_bytes(B, C, T)
    ws = torch.empty((ws_bytes + 3) // 4, device=dev, dtype=torch.float32) if ws_bytes else None
    with torch.cuda.device(dev):
        rc = lib().ema_b200_state_passing_bwd(ptr(_f32c(states)), ptr(cs_last), cs_last.stride(0),
                                              cs_last.stride(1), ptr(_f32c(dout)), ptr(dS), ptr(ddA), B, C, T,
                                              ptr(ws), ctypes.c_size_t(ws_bytes), stream_ptr(dev))
    check("ema_b200_state_passing_bwd", rc)
    dt = dout.dtype if dstates_dtype is None else dstates_dtype
    return (dS if dt == torch.float32 else dS.to(dt)), ddA


def bwd_dx(x, cs, dout, dstates, dx=None):
    dev = require_cuda(x, cs, dout, dstates, dx)
    B, L, T, C, Q = _dims(x, cs)
    res = torch.empty_like(x) if dx is None or not dx.is_contiguous() else dx
    with torch.cuda.device(dev):
        rc = lib().ema_b200_bwd_dx(ptr(_f32c(cs)), ptr(dout), ptr(_f32c(dstates)), ptr(res),
                                   dtype_code(x.dtype), B, L, T, Q, stream_ptr(dev))
    check("ema_b200_bwd_dx", rc)
    if dx is not None and res is not dx:
        dx.copy_(res)
        return dx
    return res


def _row_stage(fn_name, a, cs, b, dtype_src, raw=None):
    dev = require_cuda(a, cs, b)
    src = dtype_src
    B, L, T, C, Q = _dims(src, cs)
    out = torch.empty(B, C, Q, device=dev, dtype=torch.float32)
    fn = getattr(lib(), fn_name)
    with torch.cuda.device(dev):
        if raw is None:
            rc = fn(ptr(a), ptr(cs), ptr(b), ptr(out), dtype_code(src.dtype), B, L, T, Q, stream_ptr(dev))
        else:
            rc = fn(ptr(a), ptr(cs), ptr(b), ptr(out), dtype_code(src.dtype), int(raw), B, L, T, Q, stream_ptr(dev))
    check(fn_name, rc)
    return out


def bwd_db(x, cs, dstates, raw=False):
    return _row_stage("ema_b200_bwd_db", x, _f32c(cs), _f32c(dstates), x, raw=raw)


def bwd_dc(prev_states, cs, dout):
    return _row_stage("ema_b200_bwd_dc", _f32c(prev_states), _f32c(cs), dout, dout)


def bwd_dacs(x, cs, dout):
    return _row_stage("ema_b200_bwd_dacs", x, _f32c(cs), dout, x)
