"""ctypes binding of libema_b200.so (declarations: include/ema_b200.h)."""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_DEFAULT = os.path.join(os.path.dirname(_HERE), "lib", "libema_b200.so")

EMA_F32, EMA_BF16 = 0, 1
DECAY_PER_STEP, DECAY_PER_HEAD = 0, 1
CONV_NORTH_STAR, CONV_PRESCALED_LOG = 0, 1


class EmaB200Error(RuntimeError):
    """A libema_b200 call returned a negative status."""

    def __init__(self, fn, code, detail=""):
        self.code = code
        super().__init__(f"{fn} failed with status {code}: {detail}")


class Problem(ctypes.Structure):
    """Mirror of struct ema_b200_problem."""
    _fields_ = ([(n, ctypes.c_int64) for n in
                 ("b", "L", "h", "d", "x_sb", "x_sl", "x_sh", "y_sb", "y_sl", "y_sh",
                  "g_sb", "g_sl", "g_sh", "a_sb", "a_sl", "a_sh")] +
                [(n, ctypes.c_int32) for n in ("dtype", "decay_mode", "convention", "chunk")])


_lib = None


def lib_path():
    return os.environ.get("EMA_B200_LIB", _DEFAULT)


def lib():
    """Load the library once.  Raises if it has not been built: there is no fallback."""
    global _lib
    if _lib is not None:
        return _lib
    path = lib_path()
    if not os.path.exists(path):
        raise EmaB200Error("dlopen", -1, f"{path} not found; build it with "
                           "`python triton-kernels_b200/build.py` (set EMA_B200_LIB to override the path)")
    L = ctypes.CDLL(path)
    vp, i64, ci, cf, sz = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float, ctypes.c_size_t
    pp = ctypes.POINTER(Problem)
    sig = {
        "ema_b200_version": (ci, []),
        "ema_b200_last_cuda_error": (ci, []),
        "ema_b200_error_string": (ctypes.c_char_p, [ci]),
        "ema_b200_device_status": (ci, [ci]),
        "ema_b200_selftest_wait": (ci, [ci, ci, vp, vp]),
        "ema_b200_bounds_checked": (ci, []),
        "ema_b200_bounds_status": (ci, [ci]),
        "ema_b200_bounds_shrink_next": (ci, [sz]),
        "ema_b200_set_path": (ci, [ci]),
        "ema_b200_last_path": (ci, []),
        "ema_b200_last_schedule": (ci, []),
        "ema_b200_set_split": (ci, [ci]),
        "ema_b200_tile_steps": (ci, [pp]),
        "ema_b200_tile_states_bytes": (sz, [pp]),
        "ema_b200_bwd_workspace_bytes": (sz, [pp]),
        "ema_b200_fwd_workspace_bytes": (sz, [pp]),
        "ema_b200_fwd": (ci, [pp, vp, vp, vp, vp, vp, vp, vp, vp, cf, vp, sz, vp]),
        "ema_b200_fwd_weighted": (ci, [pp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, cf, vp, sz, vp]),
        "ema_b200_bwd": (ci, [pp, vp, vp, vp, vp, vp, vp, vp, vp, cf, vp, sz, vp]),
        "ema_b200_fold_records": (ci, [vp, ci, ci, i64, i64, ci, vp, vp]),
        "ema_b200_bwd_weighted_workspace_bytes": (sz, [pp]),
        "ema_b200_bwd_weighted": (ci, [pp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, sz, vp]),
        "ema_b200_static_scratch_limit": (sz, []),
        "ema_b200_bwd_static_scratch": (ci, [pp, vp, vp, vp, vp, vp, vp, vp]),
        "ema_b200_chunk_cumsum": (ci, [vp, i64, i64, vp, i64, i64, ci, vp]),
        "ema_b200_chunk_state": (ci, [vp, vp, vp, ci, i64, i64, i64, ci, vp]),
        "ema_b200_state_passing_fwd": (ci, [vp, vp, i64, i64, vp, vp, i64, i64, i64, vp]),
        "ema_b200_chunk_scan": (ci, [vp, vp, vp, vp, ci, i64, i64, i64, ci, vp]),
        "ema_b200_bwd_dstates": (ci, [vp, vp, vp, ci, i64, i64, i64, ci, vp]),
        "ema_b200_state_passing_bwd_workspace_bytes": (sz, [i64, i64, i64]),
        "ema_b200_state_passing_bwd": (ci, [vp, vp, i64, i64, vp, vp, vp, i64, i64, i64, vp, sz, vp]),
        "ema_b200_bwd_dx": (ci, [vp, vp, vp, vp, ci, i64, i64, i64, ci, vp]),
        "ema_b200_bwd_db": (ci, [vp, vp, vp, vp, ci, ci, i64, i64, i64, ci, vp]),
        "ema_b200_bwd_dc": (ci, [vp, vp, vp, vp, ci, i64, i64, i64, ci, vp]),
        "ema_b200_bwd_dacs": (ci, [vp, vp, vp, vp, ci, i64, i64, i64, ci, vp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args
    L._signatures = sig
    _lib = L
    return _lib


def check(fn_name, rc):
    if rc != 0:
        L = lib()
        msg = L.ema_b200_error_string(rc).decode()
        if rc == -4:
            msg += f" [cudaError {L.ema_b200_last_cuda_error()}]"
        raise EmaB200Error(fn_name, rc, msg)


def dtype_code(dt):
    if dt == torch.float32:
        return EMA_F32
    if dt == torch.bfloat16:
        return EMA_BF16
    raise TypeError(f"ema_b200 supports float32 and bfloat16 inputs, got {dt}")


def ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def stream_ptr(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def require_cuda(*tensors):
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("ema_b200 runs on CUDA tensors only (there is no CPU path)")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"tensors on different devices: {dev} and {t.device}")
    return dev
