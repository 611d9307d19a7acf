"""ema_b200: the EMA chunked scan (forward and backward) on NVIDIA B200.

PyTorch host code over a C-ABI CUDA library (libema_b200.so, hand-written sm_100a kernels).
There is no Triton, no alternative backend and no CPU path: every function here raises if the
library or a CUDA device is missing.

    from ema_b200 import ema
    y = ema(x, a)              # x[b,L,h,d], a[b,L,h] or a[h];  y_t = a_t y_{t-1} + (1-a_t) x_t
    y.backward(dy)             # dx, da

Host-resident tensors: `HostPipeline` / `ema_fwd_bwd_host` (host.py) stream batch slices through the GPU.

The reference project's own entry points (same names, same signatures) live in the sibling
package `kernels`.
"""
from ._lib import EmaB200Error, lib, lib_path  # noqa: F401
from .ops import (ema, ema_fwd, ema_bwd, ema_scan_folded_fwd, ema_scan_folded_bwd,  # noqa: F401
                  EmaFunction)
from .host import HostPipeline, bind_to_gpu_numa_node, ema_fwd_bwd_host  # noqa: F401
