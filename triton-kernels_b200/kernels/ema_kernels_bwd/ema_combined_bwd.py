"""Drop-in for kernels/ema_kernels_bwd/ema_combined_bwd.py of the reference.

The reference recomputes the forward states (3 launches), then runs six backward kernels and torch
glue, reading x three times and dout four times.  Here: one states-only forward pass over x, one
fused reverse pass over (x, dout), one small reduction.
"""
import math

import torch

from ema_b200 import ops


def _ema_chunk_scan_combined_bwd(dout, x, A, chunk_size, dt_limit=(0.0, float("inf")),
                                 recompute_output=False):
    """Returns (dx[B,L,T], ddA[B,C,Q]) and, with recompute_output, the forward output
    (reference :13-82).  ddA is the gradient of the log-decay laid out per chunk and zero padded
    past L, so that `rearrange(ddA, 'b c s -> b (c s)')[:, :L]` is dA."""
    if dout.stride(-1) != 1:
        dout = dout.contiguous()
    A = A.contiguous()
    x = x.contiguous()
    batch, seqlen, token_dim = x.shape
    nchunks = math.ceil(seqlen / chunk_size)
    assert dout.shape == (batch, seqlen, token_dim)
    assert A.shape == (batch, seqlen)

    res = ops.ema_scan_folded_bwd(dout, x, A, want_out=recompute_output)
    dx, dA = res[0], res[1]
    ddA = torch.zeros(batch, nchunks * chunk_size, device=x.device, dtype=torch.float32)
    ddA[:, :seqlen] = dA
    ddA = ddA.view(batch, nchunks, chunk_size)
    return (dx, ddA) if not recompute_output else (dx, ddA, res[2])
