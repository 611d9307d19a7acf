"""Drop-in for kernels/ema_kernels_bwd/ema_chunk_scan_chunk_state_bwd_dx.py of the reference."""
from ema_b200 import stages


def _chunk_scan_chunk_state_bwd_dx(x, dA_cumsum, dout, dstates, D=None, seq_idx=None, dx=None):
    """dx[m] = exp(min(cs_last - cs_m,0)) dstates_c + sum_{k>=m} exp(min(cs_k - cs_m,0)) dout[k]
    (reference :126-189, :208-261).  x only supplies shape and dtype, as in the reference."""
    batch, seqlen, token_dim = x.shape
    _, nchunks, chunk_size = dA_cumsum.shape
    assert dstates.shape == (batch, nchunks, token_dim)
    assert dout.shape == x.shape
    if dx is not None:
        assert dx.shape == x.shape
    return stages.bwd_dx(x, dA_cumsum, dout.contiguous(), dstates, dx=dx)
