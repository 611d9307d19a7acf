"""Drop-in for kernels/ema_kernels_bwd/ema_chunk_scan_bwd_dc.py of the reference."""
from ema_b200 import stages


def _ema_chunk_scan_bwd_dC(prev_states, dA_cumsum, dout, seq_idx=None, C=None, ngroups=1):
    """ddA_prev[b,c,m] = exp(cs_m) <dout[b, cQ+m, :], prev_states[b,c,:]>  (reference :82-112, :115-143)."""
    batch, nchunks, token_dim = prev_states.shape
    _, seqlen, _ = dout.shape
    _, _, chunk_size = dA_cumsum.shape
    assert prev_states.shape == (batch, nchunks, token_dim)
    assert dA_cumsum.shape == (batch, nchunks, chunk_size)
    assert dout.shape == (batch, seqlen, token_dim)
    return stages.bwd_dc(prev_states, dA_cumsum, dout.contiguous())
