"""Drop-in for kernels/ema_kernels/ema_cumsum.py of the reference."""
import torch

from ema_b200 import stages


def ema_chunk_cumsum_fwd(A: torch.Tensor, chunk_size: int):
    """Per-chunk inclusive cumsum of the log-decay A[B,L] -> cs[B, ceil(L/Q), Q] fp32; the ragged
    tail is padded with zeros, so cs stays constant past L (reference :57-63, :66-81)."""
    return stages.chunk_cumsum(A, chunk_size)
