"""numpy front end of the C oracle (oracle/ema_oracle.c).  TEST INFRASTRUCTURE ONLY.

`fwd` / `bwd` take dense numpy arrays x[b,L,h,d] and decay a[b,L,h] or a[h] and return what the
reference's sequential PyTorch EMA (kernels/tests/ema/test_ema_scan_fwd.py:25-37,
kernels/tests/ema_bwd/_ema_full_bwd.py:24-34) and autograd through it return.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libema_oracle.so")
_lib = None

NORTH_STAR = 0   # decay = a, x raw:      y = a y + (1-a) x
REFERENCE = 1    # decay = log a, x = u:  y = exp(A) y + u


def build(force=False):
    """Compile the C oracle with gcc (a few hundred ms)."""
    src = os.path.join(_HERE, "ema_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE])
    return _SO


def lib():
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_SO)
        i64, fp, ci = ctypes.c_int64, ctypes.c_void_p, ctypes.c_int
        L.ema_oracle_fwd.argtypes = [fp, fp, fp, fp, fp, ci, ci, ci, i64, i64, i64, i64, i64]
        L.ema_oracle_fwd.restype = ci
        L.ema_oracle_bwd.argtypes = [fp, fp, fp, fp, fp, ci, ci, ci, i64, i64, i64, i64]
        L.ema_oracle_bwd.restype = ci
        L.ema_oracle_threads.restype = ci
        L.ema_oracle_set_threads.argtypes = [ci]
        _lib = L
    return _lib


def threads():
    return int(lib().ema_oracle_threads())


def set_threads(n):
    """n worker threads over the (b,h) rows; 0 = one per online core."""
    lib().ema_oracle_set_threads(int(n))


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p) if a is not None else None


def _mode(decay, b, L, h):
    if decay.shape == (h,):
        return 1
    if decay.shape == (b, L, h):
        return 0
    raise ValueError(f"decay must be [b,L,h] or [h], got {decay.shape}")


def fwd(x, decay, convention=NORTH_STAR, chunk=0, acc64=False):
    """Returns y, or (y, chunk_start_states[b,h,C,d], final_state[b,h,d]) when chunk > 0."""
    x = _f32(x)
    decay = _f32(decay)
    b, L, h, d = x.shape
    mode = _mode(decay, b, L, h)
    y = np.empty_like(x)
    states = final = None
    if chunk > 0:
        C = (L + chunk - 1) // chunk
        states = np.zeros((b, h, C, d), np.float32)
        final = np.zeros((b, h, d), np.float32)
    rc = lib().ema_oracle_fwd(_ptr(x), _ptr(decay), _ptr(y), _ptr(states), _ptr(final), mode,
                              convention, int(acc64), b, L, h, d, chunk)
    assert rc == 0
    return (y, states, final) if chunk > 0 else y


def bwd(x, decay, dy, convention=NORTH_STAR, acc64=False):
    """Returns (dx[b,L,h,d], ddecay shaped like decay)."""
    x = _f32(x)
    decay = _f32(decay)
    dy = _f32(dy)
    b, L, h, d = x.shape
    mode = _mode(decay, b, L, h)
    dx = np.empty_like(x)
    dd = np.zeros_like(decay)
    rc = lib().ema_oracle_bwd(_ptr(x), _ptr(decay), _ptr(dy), _ptr(dx), _ptr(dd), mode, convention,
                              int(acc64), b, L, h, d)
    assert rc == 0
    return dx, dd
