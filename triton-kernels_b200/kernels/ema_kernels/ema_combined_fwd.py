"""Drop-in for kernels/ema_kernels/ema_combined_fwd.py of the reference.

The reference chains four launches (cumsum, chunk state, state passing, scan) and reads X twice;
here one fused kernel reads X once and emits the output, the chunk-start states and the final
state together; the tiny cumsum is produced by its own stage kernel because callers get it back.
"""
import torch

from ema_b200 import ops
from kernels.ema_kernels.ema_cumsum import ema_chunk_cumsum_fwd


def _ema_matmul_scan_combined_fwd(A_ema, X_ema, chunk_size, dtype=torch.float32):
    """(out[B,L,T], cs[B,C,Q], chunk_start_states[B,C,T], final_state[B,T]) - reference :12-47."""
    ema_cs = ema_chunk_cumsum_fwd(A_ema, chunk_size=chunk_size)
    out, states, final = ops.ema_scan_folded_fwd(A_ema, X_ema, chunk_size)
    if dtype != torch.float32:
        states = states.to(dtype)
    return out, ema_cs, states, final


class EMAMatmulCombinedFn(torch.autograd.Function):
    """Same forward as the reference's class (:51-61).  The reference's backward is a stub that
    returns None; this one returns the gradients of (A_ema, X_ema)."""

    @staticmethod
    def forward(ctx, A_ema, X_ema, chunk_size):
        r = ops.ema_fwd(X_ema.unsqueeze(2), A_ema.unsqueeze(2), prescaled_log=True, want_tile_states=True)
        ctx.save_for_backward(A_ema, X_ema, r["tile_states"])
        ctx.chunk_size = chunk_size
        return r["y"].squeeze(2)

    @staticmethod
    def backward(ctx, dout, *args):
        A_ema, X_ema, tile_states = ctx.saved_tensors
        r = ops.ema_bwd(X_ema.unsqueeze(2), A_ema.unsqueeze(2), dout.unsqueeze(2), tile_states,
                        prescaled_log=True)
        return r["ddecay"].squeeze(2).to(A_ema.dtype), r["dx"].squeeze(2), None


def ema_matmul_scan_combined(A_ema, X_ema, chunk_size):
    return EMAMatmulCombinedFn.apply(A_ema, X_ema, chunk_size)
