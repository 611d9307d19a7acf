"""The binding a maintainer of the reference project would add: ctypes stubs that hand the tensors' device pointers to
libema_b200.so, for the combined forward (kernels/ema_kernels/ema_combined_fwd.py:12 of the reference) and for the
heads-style entry point without gradients (kernels/ema_combined.py:100, state size 1).  In the reference this would be
a new file kernels/ema_kernels/_b200.py; the other entry points follow the same pattern with the argument lists of
include/ema_b200.h.  ema_b200/_lib.py is the complete version (all entry points, error mapping).

The library is looked up in $EMA_B200_LIB, then next to this package (triton-kernels_b200/lib/), then on the loader's
search path.
"""
import ctypes
import os

import torch

_here = os.path.dirname(os.path.abspath(__file__))
_candidates = [os.environ.get("EMA_B200_LIB"), os.path.join(os.path.dirname(_here), "lib", "libema_b200.so")]
_lib = ctypes.CDLL(next((c for c in _candidates if c and os.path.exists(c)), "libema_b200.so"))


class _Problem(ctypes.Structure):            # struct ema_b200_problem
    _fields_ = [(n, ctypes.c_int64) for n in
                ("b", "L", "h", "d", "x_sb", "x_sl", "x_sh", "y_sb", "y_sl", "y_sh",
                 "g_sb", "g_sl", "g_sh", "a_sb", "a_sl", "a_sh")] + \
               [(n, ctypes.c_int) for n in ("dtype", "decay_mode", "convention", "chunk")]

_lib.ema_b200_fwd.restype = ctypes.c_int
_lib.ema_b200_fwd.argtypes = ([ctypes.POINTER(_Problem)] + [ctypes.c_void_p] * 8 +
                                 [ctypes.c_float, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p])
_lib.ema_b200_error_string.restype = ctypes.c_char_p

def _p(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())

def ema_matmul_scan_combined_fwd(A_ema, X_ema, chunk_size):
    """A_ema[B, L] = log decay, X_ema[B, L, T] pre-scaled input -> (out, chunk-start states, final state)."""
    B, L, T = X_ema.shape
    C = (L + chunk_size - 1) // chunk_size
    A32 = A_ema.float().contiguous()
    out = torch.empty_like(X_ema)
    states = torch.empty((B, C, T), dtype=torch.float32, device=X_ema.device)
    final = torch.empty((B, T), dtype=torch.float32, device=X_ema.device)
    p = _Problem(b=B, L=L, h=1, d=T,
                 x_sb=X_ema.stride(0), x_sl=X_ema.stride(1), x_sh=0,
                 y_sb=out.stride(0), y_sl=out.stride(1), y_sh=0,
                 g_sb=0, g_sl=0, g_sh=0, a_sb=A32.stride(0), a_sl=A32.stride(1), a_sh=0,
                 dtype=0 if X_ema.dtype == torch.float32 else 1,      # EMA_F32 / EMA_BF16
                 decay_mode=0, convention=1, chunk=chunk_size)        # per-step decay, pre-scaled log convention
    stream = ctypes.c_void_p(torch.cuda.current_stream(X_ema.device).cuda_stream)
    with torch.cuda.device(X_ema.device):
        rc = _lib.ema_b200_fwd(ctypes.byref(p), _p(X_ema), _p(A32), _p(out), _p(states), None, None, _p(final), None,
                               ctypes.c_float(0.0), None, 0, stream)      # no scratch: see "workspace" in the header
    if rc:
        raise RuntimeError(_lib.ema_b200_error_string(rc).decode())
    return out, states, final


_lib.ema_b200_fwd_weighted.restype = ctypes.c_int
_lib.ema_b200_fwd_weighted.argtypes = ([ctypes.POINTER(_Problem)] + [ctypes.c_void_p] * 10 +
                                          [ctypes.c_float, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p])

def ema_chunk_scan_combined_inference(x, dt, A, B, C):
    """x[b, l, h, p]; dt[b, l, h] already processed (bias, softplus, limits); A[h]; B, C[b, l, h] (state size 1)."""
    b, l, h, d = x.shape
    a_log = (dt * A).float().contiguous()          # log decay per step
    w_in = (dt * B).float().contiguous()           # input weight
    w_out = C.float().contiguous()                 # output weight
    out = torch.empty_like(x)
    p = _Problem(b=b, L=l, h=h, d=d, x_sb=x.stride(0), x_sl=x.stride(1), x_sh=x.stride(2),
                 y_sb=out.stride(0), y_sl=out.stride(1), y_sh=out.stride(2), g_sb=0, g_sl=0, g_sh=0,
                 a_sb=a_log.stride(0), a_sl=a_log.stride(1), a_sh=a_log.stride(2),
                 dtype=0 if x.dtype == torch.float32 else 1, decay_mode=0, convention=1, chunk=0)
    stream = ctypes.c_void_p(torch.cuda.current_stream(x.device).cuda_stream)
    with torch.cuda.device(x.device):
        rc = _lib.ema_b200_fwd_weighted(ctypes.byref(p), _p(x), _p(a_log), _p(w_in), _p(w_out), _p(out),
                                        None, None, None, None, None, ctypes.c_float(0.0), None, 0, stream)
    if rc:
        raise RuntimeError(_lib.ema_b200_error_string(rc).decode())
    return out
