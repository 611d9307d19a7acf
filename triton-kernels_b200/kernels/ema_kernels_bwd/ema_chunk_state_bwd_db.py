"""Drop-in for kernels/ema_kernels_bwd/ema_chunk_state_bwd_db.py of the reference."""
from ema_b200 import stages


def _ema_chunk_state_bwd_db(x, dA_cumsum, dstates, seq_idx=None, B=None, ngroups=1,
                            raw_scale_gradient=False):
    """Decay gradient through the chunk state: g_m = exp(min(cs_last - cs_m,0)) <dstates_c, x_m>
    stored at slot m+1, then summed along the chunk unless raw_scale_gradient
    (reference :75-117, :122-153).  Plain stores replace the reference's float atomics."""
    batch, seqlen, token_dim = x.shape
    _, nchunks, chunk_size = dA_cumsum.shape
    assert dstates.shape == (batch, nchunks, token_dim)
    return stages.bwd_db(x.contiguous(), dA_cumsum, dstates, raw=raw_scale_gradient)
