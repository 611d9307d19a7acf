"""Host side of the fused EMA scan: tensor checks, output allocation, C-ABI calls, autograd.

Layouts follow the reference project's heads-style convention (kernels/ema_combined.py:100:
x[b, l, h, p] with one decay per (b, l, h) or per head): x[b, L, h, d], decay a[b, L, h] or a[h].
The reference's folded layout X[B, L, T] with A[B, L] is the same thing with h = 1.
"""
import ctypes
import json
import os

import torch

from . import _lib
from ._lib import (CONV_NORTH_STAR, CONV_PRESCALED_LOG, DECAY_PER_HEAD, DECAY_PER_STEP, Problem,
                   check, dtype_code, lib, ptr, require_cuda, stream_ptr)


class _traced:
    """Optional tracing of a library call, off by default.  EMA_B200_NVTX=1 wraps the call in an NVTX range (visible in
    a profiler's timeline); EMA_B200_TRACE=<file> appends one JSON line per call - op, shape, dtype, decay mode, kernel
    family and schedule, milliseconds between two CUDA events around the call, and the GB/s and tokens/s that follow
    from the algorithmic bytes (x read + y written forward; x, dy read + dx written backward).  Tracing a call
    synchronises the device, so it is a debugging aid, not for timed runs."""

    def __init__(self, op, x, decay, passes):
        self.op, self.x, self.decay, self.passes = op, x, decay, passes
        self.nvtx = os.environ.get("EMA_B200_NVTX") == "1"
        self.path = os.environ.get("EMA_B200_TRACE")

    def __enter__(self):
        if self.nvtx:
            torch.cuda.nvtx.range_push(f"ema_b200.{self.op} {tuple(self.x.shape)}")
        if self.path:
            self.e0, self.e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self.e0.record(torch.cuda.current_stream(self.x.device))
        return self

    def __exit__(self, *exc):
        if self.path and exc[0] is None:
            self.e1.record(torch.cuda.current_stream(self.x.device))
            self.e1.synchronize()
            ms = self.e0.elapsed_time(self.e1)
            b, L, h, d = self.x.shape
            nbytes = self.passes * self.x.numel() * self.x.element_size() + self.decay.numel() * 4
            rec = {"op": self.op, "shape": [b, L, h, d], "dtype": str(self.x.dtype).replace("torch.", ""),
                   "decay": "per_head" if self.decay.dim() == 1 else "per_step", "path": lib().ema_b200_last_path(),
                   "schedule": lib().ema_b200_last_schedule(), "ms": ms,
                   "algorithmic_GBps": nbytes / (ms * 1e-3) / 1e9 if ms > 0 else None,
                   "tokens_per_s": b * L / (ms * 1e-3) if ms > 0 else None}
            with open(self.path, "a") as f:
                f.write(json.dumps(rec) + "\n")
        if self.nvtx:
            torch.cuda.nvtx.range_pop()
        return False


def _problem(x, decay, out, dy=None, convention=CONV_NORTH_STAR, chunk=0):
    b, L, h, d = x.shape
    p = Problem()
    p.b, p.L, p.h, p.d = b, L, h, d
    p.x_sb, p.x_sl, p.x_sh = x.stride(0), x.stride(1), x.stride(2)
    p.y_sb, p.y_sl, p.y_sh = out.stride(0), out.stride(1), out.stride(2)
    if dy is not None:
        p.g_sb, p.g_sl, p.g_sh = dy.stride(0), dy.stride(1), dy.stride(2)
    if decay.dim() == 1:
        p.decay_mode = DECAY_PER_HEAD
        p.a_sh = decay.stride(0)
    else:
        p.decay_mode = DECAY_PER_STEP
        p.a_sb, p.a_sl, p.a_sh = decay.stride(0), decay.stride(1), decay.stride(2)
    p.dtype = dtype_code(x.dtype)
    p.convention = convention
    p.chunk = int(chunk)
    return p


def _check_inputs(x, decay):
    if x.dim() != 4:
        raise ValueError(f"x must be [b, L, h, d], got shape {tuple(x.shape)}")
    b, L, h, d = x.shape
    if decay.dim() == 1:
        if decay.shape[0] != h:
            raise ValueError(f"per-head decay must have shape [{h}], got {tuple(decay.shape)}")
    elif tuple(decay.shape) != (b, L, h):
        raise ValueError(f"decay must be [b, L, h] = {(b, L, h)} or [h], got {tuple(decay.shape)}")
    if x.stride(-1) != 1 and d > 1:
        x = x.contiguous()
    if decay.dtype != torch.float32:
        decay = decay.float()
    return x, decay


def _check_device_status(dev):
    """Reads and clears the device status word (synchronises `dev`); raises if a bounded wait ran out."""
    with torch.cuda.device(dev):
        check("ema_b200_device_status", lib().ema_b200_device_status(1))


def n_tiles_of(x, decay, convention=CONV_NORTH_STAR):
    """(tile_steps, n_tiles) the library uses for this problem."""
    p = _problem(x, decay, x, convention=convention)
    ts = lib().ema_b200_tile_steps(ctypes.byref(p))
    if ts <= 0:
        raise _lib.EmaB200Error("ema_b200_tile_steps", -3, "unsupported problem")
    return ts, (x.shape[1] + ts - 1) // ts


def ema_fwd(x, decay, *, chunk=0, prescaled_log=False, init_state=None, want_chunk_states=False,
            want_tile_states=False, want_final=False, want_log_decay_sum=False, stop_below=0.0,
            out=None, tile_states=None, workspace=None, in_weight=None, out_weight=None, final_out=None,
            log_decay_sum_out=None, check_status=False):
    """Forward scan.  Returns a dict with 'y' and the requested extras.

    x[b,L,h,d] (fp32|bf16, last dim contiguous), decay a[b,L,h] or a[h] (fp32).
    prescaled_log=True selects the reference's (A_ema, X_ema) convention: decay = log a, x = (1-a) x.
    `out` / `tile_states` let a caller re-scan a prefix in place (sequence-parallel fix-up).
    `workspace` (returned as 'fwd_workspace') is the small scratch that lets the kernels spread uneven work
    over all SMs; pass it back in to avoid the allocation, never to two calls that may overlap.
    `in_weight` / `out_weight` (fp32 [b,L,h], per-step decay only) fold per-step weights into the same pass:
    s_t = a_t s_{t-1} + in_weight_t x_t, y_t = out_weight_t s_t; the returned states are the s themselves.
    `final_out` (fp32 [b,h,d]) / `log_decay_sum_out` (fp32 [b,h]), both contiguous, receive the final state and the
    summed log decay in place (e.g. two views of one buffer that is then sent to other ranks).
    `check_status=True` reads the device status word after the call (this synchronises the device) and raises
    EmaB200Error(EMA_ERR_TIMEOUT) if a bounded device-side wait ran out.
    """
    x, decay = _check_inputs(x, decay)
    dev = require_cuda(x, decay, init_state, out, tile_states, in_weight, out_weight)
    b, L, h, d = x.shape
    weighted = in_weight is not None or out_weight is not None
    if weighted:
        if decay.dim() != 3:
            raise ValueError("per-step weights need a per-step decay [b, L, h]")
        decay = decay.contiguous()

        def _as_weight(w, name):
            if w is None:
                return None
            if tuple(w.shape) != (b, L, h) or w.dtype != torch.float32:
                raise ValueError(f"{name} must be fp32 [b, L, h]")
            return w.contiguous()   # the kernels index the weights with the decay's strides
        in_weight, out_weight = _as_weight(in_weight, "in_weight"), _as_weight(out_weight, "out_weight")
    conv = CONV_PRESCALED_LOG if prescaled_log else CONV_NORTH_STAR
    y = out if out is not None else torch.empty((b, L, h, d), dtype=x.dtype, device=dev)
    p = _problem(x, decay, y, convention=conv, chunk=chunk)
    L_ = lib()
    res = {"y": y}
    cs = ts = fin = lds = None
    if want_chunk_states:
        if chunk <= 0:
            raise ValueError("chunk must be positive to return chunk states")
        cs = torch.empty((b, h, (L + chunk - 1) // chunk, d), dtype=torch.float32, device=dev)
        res["chunk_states"] = cs
    if want_tile_states or tile_states is not None:
        tsteps = L_.ema_b200_tile_steps(ctypes.byref(p))
        nt = (L + tsteps - 1) // tsteps if tsteps > 0 else 0
        ts = tile_states if tile_states is not None else torch.empty((b * h, nt, d), dtype=torch.float32, device=dev)
        res["tile_states"] = ts
    if want_final or final_out is not None:
        fin = final_out if final_out is not None else torch.empty((b, h, d), dtype=torch.float32, device=dev)
        if tuple(fin.shape) != (b, h, d) or fin.dtype != torch.float32 or not fin.is_contiguous():
            raise ValueError("final_out must be contiguous fp32 [b, h, d]")
        res["final_state"] = fin
    if want_log_decay_sum or log_decay_sum_out is not None:
        lds = log_decay_sum_out if log_decay_sum_out is not None else torch.zeros((b, h), dtype=torch.float32, device=dev)
        if tuple(lds.shape) != (b, h) or lds.dtype != torch.float32 or not lds.is_contiguous():
            raise ValueError("log_decay_sum_out must be contiguous fp32 [b, h]")
        res["log_decay_sum"] = lds
    if init_state is not None:
        if tuple(init_state.shape) != (b, h, d) or init_state.dtype != torch.float32:
            raise ValueError("init_state must be fp32 [b, h, d]")
        init_state = init_state.contiguous()
    ws_bytes = L_.ema_b200_fwd_workspace_bytes(ctypes.byref(p))
    if workspace is None and ws_bytes > 0:
        workspace = torch.empty(((ws_bytes + 3) // 4,), dtype=torch.float32, device=dev)
    res["fwd_workspace"] = workspace
    ws_size = ctypes.c_size_t(0 if workspace is None else workspace.numel() * 4)
    with torch.cuda.device(dev), _traced("ema_fwd", x, decay, 2):
        if weighted:
            rc = L_.ema_b200_fwd_weighted(ctypes.byref(p), ptr(x), ptr(decay), ptr(in_weight), ptr(out_weight), ptr(y),
                                          ptr(cs), ptr(ts), ptr(init_state), ptr(fin), ptr(lds),
                                          ctypes.c_float(stop_below), ptr(workspace), ws_size, stream_ptr(dev))
        else:
            rc = L_.ema_b200_fwd(ctypes.byref(p), ptr(x), ptr(decay), ptr(y), ptr(cs), ptr(ts), ptr(init_state),
                                 ptr(fin), ptr(lds), ctypes.c_float(stop_below), ptr(workspace), ws_size,
                                 stream_ptr(dev))
    check("ema_b200_fwd_weighted" if weighted else "ema_b200_fwd", rc)
    if check_status:
        _check_device_status(dev)
    return res


def ema_bwd(x, decay, dy, tile_states, *, prescaled_log=False, dfinal_state=None, want_dinit=False,
            stop_below=0.0, dx=None, workspace=None, ddecay=None, dinit_out=None, check_status=False):
    """Backward scan.  Returns a dict with 'dx', 'ddecay' (shaped like decay) and optionally 'dinit_state'.

    `dx`, `workspace`, `ddecay` let a caller re-scan a suffix in place (sequence-parallel fix-up):
    the workspace keeps the partial sums of the first pass, so it must be the same tensor.
    """
    x, decay = _check_inputs(x, decay)
    if dy.shape != x.shape or dy.dtype != x.dtype:
        raise ValueError("dy must match x in shape and dtype")
    if dy.stride(-1) != 1 and dy.shape[-1] > 1:
        dy = dy.contiguous()
    decay = decay.contiguous()
    dev = require_cuda(x, decay, dy, tile_states, dfinal_state)
    b, L, h, d = x.shape
    conv = CONV_PRESCALED_LOG if prescaled_log else CONV_NORTH_STAR
    if dx is None:
        dx = torch.empty((b, L, h, d), dtype=x.dtype, device=dev)
    if ddecay is None:
        ddecay = torch.empty_like(decay)
    p = _problem(x, decay, dx, dy=dy, convention=conv)
    L_ = lib()
    nbytes = L_.ema_b200_bwd_workspace_bytes(ctypes.byref(p))
    if workspace is None:
        workspace = torch.empty(((nbytes + 3) // 4,), dtype=torch.float32, device=dev)
    dinit = None
    if want_dinit or dinit_out is not None:
        dinit = dinit_out if dinit_out is not None else torch.empty((b, h, d), dtype=torch.float32, device=dev)
        if tuple(dinit.shape) != (b, h, d) or dinit.dtype != torch.float32 or not dinit.is_contiguous():
            raise ValueError("dinit_out must be contiguous fp32 [b, h, d]")
    if dfinal_state is not None:
        if tuple(dfinal_state.shape) != (b, h, d) or dfinal_state.dtype != torch.float32:
            raise ValueError("dfinal_state must be fp32 [b, h, d]")
        dfinal_state = dfinal_state.contiguous()
    with torch.cuda.device(dev), _traced("ema_bwd", x, decay, 3):
        rc = L_.ema_b200_bwd(ctypes.byref(p), ptr(x), ptr(decay), ptr(dy), ptr(tile_states), ptr(dx),
                             ptr(ddecay), ptr(dfinal_state), ptr(dinit), ctypes.c_float(stop_below),
                             ptr(workspace), ctypes.c_size_t(workspace.numel() * 4), stream_ptr(dev))
    check("ema_b200_bwd", rc)
    if check_status:
        _check_device_status(dev)
    res = {"dx": dx, "ddecay": ddecay, "workspace": workspace}
    if dinit is not None:
        res["dinit_state"] = dinit
    return res


def ema_bwd_weighted(x, decay, dy, tile_states, *, in_weight=None, out_weight=None, prescaled_log=False,
                     dfinal_state=None, want_dinit=False):
    """Backward of the weighted forward scan (ema_fwd with in_weight / out_weight), one pass over x and dy.

    Returns a dict with 'dx', 'ddecay' and, for the weights that were given, 'din_weight' / 'dout_weight' (fp32
    [b, L, h]); optionally 'dinit_state'.  Per-step decay only; `tile_states` are the ones the weighted forward saved.
    """
    x, decay = _check_inputs(x, decay)
    if decay.dim() != 3:
        raise ValueError("per-step weights need a per-step decay [b, L, h]")
    if dy.shape != x.shape or dy.dtype != x.dtype:
        raise ValueError("dy must match x in shape and dtype")
    if dy.stride(-1) != 1 and dy.shape[-1] > 1:
        dy = dy.contiguous()
    decay = decay.contiguous()
    dev = require_cuda(x, decay, dy, tile_states, dfinal_state, in_weight, out_weight)
    b, L, h, d = x.shape

    def _as_weight(w, name):
        if w is None:
            return None
        if tuple(w.shape) != (b, L, h) or w.dtype != torch.float32:
            raise ValueError(f"{name} must be fp32 [b, L, h]")
        return w.contiguous()
    in_weight, out_weight = _as_weight(in_weight, "in_weight"), _as_weight(out_weight, "out_weight")
    conv = CONV_PRESCALED_LOG if prescaled_log else CONV_NORTH_STAR
    dx = torch.empty((b, L, h, d), dtype=x.dtype, device=dev)
    ddecay = torch.empty_like(decay)
    dw = torch.empty_like(decay) if in_weight is not None else None
    dc = torch.empty_like(decay) if out_weight is not None else None
    p = _problem(x, decay, dx, dy=dy, convention=conv)
    L_ = lib()
    nbytes = L_.ema_b200_bwd_weighted_workspace_bytes(ctypes.byref(p))
    workspace = torch.empty(((nbytes + 3) // 4,), dtype=torch.float32, device=dev)
    dinit = torch.empty((b, h, d), dtype=torch.float32, device=dev) if want_dinit else None
    if dfinal_state is not None:
        if tuple(dfinal_state.shape) != (b, h, d) or dfinal_state.dtype != torch.float32:
            raise ValueError("dfinal_state must be fp32 [b, h, d]")
        dfinal_state = dfinal_state.contiguous()
    with torch.cuda.device(dev), _traced("ema_bwd_weighted", x, decay, 3):
        rc = L_.ema_b200_bwd_weighted(ctypes.byref(p), ptr(x), ptr(decay), ptr(in_weight), ptr(out_weight), ptr(dy),
                                      ptr(tile_states), ptr(dx), ptr(ddecay), ptr(dw), ptr(dc), ptr(dfinal_state),
                                      ptr(dinit), ptr(workspace), ctypes.c_size_t(workspace.numel() * 4), stream_ptr(dev))
    check("ema_b200_bwd_weighted", rc)
    res = {"dx": dx, "ddecay": ddecay}
    if dw is not None:
        res["din_weight"] = dw
    if dc is not None:
        res["dout_weight"] = dc
    if dinit is not None:
        res["dinit_state"] = dinit
    return res


def fold_records(records, rank, rows, d, reverse=False, out=None):
    """State (reverse=False) or adjoint (reverse=True) entering segment `rank`, folded from the gathered
    per-rank records [world, rows*d + rows] = [zero-state final (or dinit) | summed log decay]."""
    dev = require_cuda(records, out)
    if records.dtype != torch.float32 or records.dim() != 2 or records.shape[1] != rows * d + rows or \
            not records.is_contiguous():
        raise ValueError("records must be contiguous fp32 [world, rows*d + rows]")
    if out is None:
        out = torch.empty((rows, d), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        rc = lib().ema_b200_fold_records(ptr(records), int(records.shape[0]), int(rank), rows, d,
                                         1 if reverse else 0, ptr(out), stream_ptr(dev))
    check("ema_b200_fold_records", rc)
    return out


def ema_bwd_static_scratch(x, decay, dy, tile_states, dx, ddecay, *, prescaled_log=False):
    """Backward scan into caller-provided `dx` and `ddecay`, with no allocation of any kind.

    The partial sums of the decay gradient go to a fixed array inside the library (one per device,
    `static_scratch_limit()` bytes); problems that need more raise EmaB200Error.  For callers that must
    not enter torch's allocator or cudaMalloc at the time of the call.  Every tensor must already have
    the layout the library wants (unit stride on d, contiguous decay): nothing is copied here.  Calls
    on one device must not overlap (same stream, or ordered by events): they share the array.  Make
    the first call on a device at start-up, outside any stream capture: it does the one-time set-up.
    """
    if dy.shape != x.shape or dy.dtype != x.dtype or dx.shape != x.shape or dx.dtype != x.dtype:
        raise ValueError("dy and dx must match x in shape and dtype")
    if any(t.stride(-1) != 1 and t.shape[-1] > 1 for t in (x, dy, dx)) or not decay.is_contiguous():
        raise ValueError("x, dy, dx need unit stride on d and decay must be contiguous")
    if decay.dtype != torch.float32 or ddecay.dtype != torch.float32 or ddecay.shape != decay.shape:
        raise ValueError("decay and ddecay must be fp32 and of one shape")
    dev = require_cuda(x, decay, dy, tile_states, dx, ddecay)
    conv = CONV_PRESCALED_LOG if prescaled_log else CONV_NORTH_STAR
    p = _problem(x, decay, dx, dy=dy, convention=conv)
    with torch.cuda.device(dev):
        rc = lib().ema_b200_bwd_static_scratch(ctypes.byref(p), ptr(x), ptr(decay), ptr(dy), ptr(tile_states),
                                               ptr(dx), ptr(ddecay), stream_ptr(dev))
    check("ema_b200_bwd_static_scratch", rc)
    return dx, ddecay


def static_scratch_limit():
    """Bytes of the library's built-in scratch array (the limit of ema_bwd_static_scratch)."""
    return int(lib().ema_b200_static_scratch_limit())


class EmaFunction(torch.autograd.Function):
    """y_t = a_t y_{t-1} + (1 - a_t) x_t with gradients for x and a."""

    @staticmethod
    def forward(ctx, x, a):
        r = ema_fwd(x, a, want_tile_states=True)
        ctx.save_for_backward(x, a, r["tile_states"])
        return r["y"]

    @staticmethod
    def backward(ctx, dy):
        x, a, tile_states = ctx.saved_tensors
        r = ema_bwd(x, a, dy, tile_states)
        da = r["ddecay"]
        return r["dx"], (da.to(a.dtype) if da.dtype != a.dtype else da)


def ema(x, a):
    """EMA over the sequence axis of x[b, L, h, d] with decay a[b, L, h] or a[h]; differentiable."""
    return EmaFunction.apply(x, a)


# ---- the reference's folded layout ------------------------------------------------------------

def ema_scan_folded_fwd(A, X, chunk_size, want_states=True):
    """(out[B,L,T], chunk_start_states[B,C,T] fp32, final[B,T] fp32) for A[B,L] = log a, X[B,L,T] = u.

    Same quantities as _ema_matmul_scan_combined_fwd (kernels/ema_kernels/ema_combined_fwd.py:12-47).
    """
    if X.dim() != 3 or A.dim() != 2 or A.shape != X.shape[:2]:
        raise ValueError(f"expected X[B,L,T] and A[B,L], got {tuple(X.shape)} and {tuple(A.shape)}")
    r = ema_fwd(X.unsqueeze(2), A.unsqueeze(2), chunk=chunk_size, prescaled_log=True,
                want_chunk_states=want_states, want_final=True)
    states = r["chunk_states"].squeeze(1) if want_states else None
    return r["y"].squeeze(2), states, r["final_state"].squeeze(1)


def ema_scan_folded_bwd(dout, X, A, want_out=False):
    """(dX[B,L,T], dA[B,L] fp32[, out]) for the folded layout; the forward states are recomputed."""
    X4, A4 = X.unsqueeze(2), A.unsqueeze(2)
    f = ema_fwd(X4, A4, prescaled_log=True, want_tile_states=True)
    r = ema_bwd(X4, A4, dout.unsqueeze(2), f["tile_states"], prescaled_log=True)
    res = (r["dx"].squeeze(2), r["ddecay"].squeeze(2))
    return res + (f["y"].squeeze(2),) if want_out else res
