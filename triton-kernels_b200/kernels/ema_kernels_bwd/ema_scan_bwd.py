"""Drop-in for kernels/ema_kernels_bwd/ema_scan_bwd.py of the reference."""
from ema_b200 import stages


def _ema_chunk_scan_bwd_dstates(dA_cumsum, dout, seq_idx=None, dtype=None):
    """dprev_states[b,c,:] = sum_q exp(cs_q) dout[b, cQ+q, :]  (reference :96-110, :132-152)."""
    batch, seqlen, token_dim = dout.shape
    _, nchunks, chunk_size = dA_cumsum.shape
    assert dA_cumsum.shape == (batch, nchunks, chunk_size)
    return stages.bwd_dstates(dA_cumsum, dout, dtype=dtype)
