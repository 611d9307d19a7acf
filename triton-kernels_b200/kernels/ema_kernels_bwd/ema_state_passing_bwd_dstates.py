"""Drop-in for kernels/ema_kernels_bwd/ema_state_passing_bwd_dstates.py of the reference."""
from ema_b200 import stages


def _ema_state_passing_bwd(states, dA_chunk_cumsum, dout, dfinal_states=None, seq_idx=None,
                           has_initial_states=False, dstates_dtype=None, states_dtype=None,
                           chunk_size=None):
    """Reverse carry of the adjoint over chunks (reference :60-98, :103-184).

    Returns (dstates[B,C,T], ddA_chunk_cumsum[B,C], None).  The sum over the channel dimension is
    done inside one CTA per batch row, so the per-block partial buffer of the reference (sized for
    64-wide blocks while its kernel runs 16-wide ones) does not exist here."""
    batch, nchunks, token_dim = states.shape
    assert dA_chunk_cumsum.shape == (batch, nchunks)
    assert dout.shape == (batch, nchunks, token_dim)
    assert dfinal_states is None
    assert seq_idx is None
    assert not has_initial_states
    dstates, ddA = stages.state_passing_bwd(states, dA_chunk_cumsum, dout, dstates_dtype=dstates_dtype)
    return dstates, ddA.to(dA_chunk_cumsum.dtype), None
