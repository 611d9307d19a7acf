"""Drop-in for kernels/ema_kernels_bwd/ema_scan_da.py of the reference."""
from ema_b200 import stages


def _ema_chunk_scan_bwd_ddAcs_stable(x, dA_cumsum, dout):
    """Intra-chunk decay gradient: out[j+1] = sum_{m>j} sum_{k<=j} <dout_m, x_k> exp(min(cs_m-cs_k,0)),
    out[0] = 0 (reference :69-106, :113-137).  Computed with two O(Q) scans per channel instead of
    the Q x Q product, and without the [B,C,Q/16,Q] partial buffer."""
    batch, seqlen, token_dim = x.shape
    assert dout.shape == x.shape
    return stages.bwd_dacs(x.contiguous(), dA_cumsum, dout.contiguous())
