"""Drop-in for kernels/ema_kernels/ema_state_pass.py of the reference."""
import torch

from ema_b200 import stages


def _ema_state_passing_fwd(states: torch.Tensor, A_cs_last: torch.Tensor, initial_states=None,
                           chunk_size=None, out_dtype=None):
    """Serial carry over chunks: returns (state at the START of every chunk [B,C,T], final state
    [B,T] fp32); chunk 0 starts from zeros (reference :100-120, :125-155)."""
    batch, nchunks, token_dim = states.shape
    assert A_cs_last.shape == (batch, nchunks)
    if initial_states is not None:
        raise NotImplementedError("No support for init_states in EMA kernel.")
    return stages.state_passing_fwd(states, A_cs_last, out_dtype=out_dtype)
