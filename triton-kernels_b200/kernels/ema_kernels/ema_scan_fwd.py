"""Drop-in for kernels/ema_kernels/ema_scan_fwd.py of the reference."""
from ema_b200 import stages


def _ema_scan_fwd(x, A_cumsum, states):
    """out[m] = exp(min(cs_m,0)) states_c + sum_{k<=m} exp(min(cs_m - cs_k,0)) x[k], per chunk
    (reference :111-156, :161-193).  Output has x's dtype; rows past L do not exist."""
    return stages.chunk_scan(x, A_cumsum, states)
