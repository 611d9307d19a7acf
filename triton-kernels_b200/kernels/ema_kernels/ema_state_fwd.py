"""Drop-in for kernels/ema_kernels/ema_state_fwd.py of the reference."""
import math

from ema_b200 import stages


def _ema_chunk_state_fwd(x, A_cumsum, seq_idx=None, states=None, states_in_fp32=True):
    """S[b,c,:] = sum_q exp(min(cs_last - cs_q, 0)) x[b, cQ+q, :]  (reference :130-163).
    `seq_idx` is accepted and ignored, as in the reference."""
    batch, seqlen, token_dim = x.shape
    _, _, chunk_size = A_cumsum.shape
    nchunks = math.ceil(seqlen / chunk_size)
    assert x.is_contiguous()
    assert A_cumsum.is_contiguous()
    assert A_cumsum.shape == (batch, nchunks, chunk_size)
    if states is not None:
        assert states.shape == (batch, nchunks, token_dim)
    return stages.chunk_state(x, A_cumsum, states=states, states_in_fp32=states_in_fp32)
