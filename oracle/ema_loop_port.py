"""The reference's CPU path, restated: sequential PyTorch EMA loops.  TEST INFRASTRUCTURE ONLY.

These are the loops the reference project runs on the CPU as its own ground truth
(kernels/tests/ema/test_ema_scan_fwd.py:25-37 p-weighted; kernels/tests/ema_bwd/_ema_full_bwd.py:24-34
pre-scaled): a Python loop over batch rows and time steps with a torch vector op over the channel
dimension per step, gradients by autograd through the loop.  bench.py times them as the CPU
reference arm; they are Python-interpreter bound by construction, like the original.
"""
import torch


def ema_loop_pweighted(X, P):
    """X[B,T,D], P[B,T,1] -> Z[B,T,D];  z_t = (1-p_t) z_{t-1} + p_t x_t."""
    B, T, D = X.shape
    rows = []
    for b in range(B):
        z_prev = torch.zeros(D, dtype=X.dtype)
        steps = []
        for t in range(T):
            p = P[b, t, 0]
            z_prev = (1.0 - p) * z_prev + p * X[b, t]
            steps.append(z_prev)
        rows.append(torch.stack(steps))
    return torch.stack(rows)


def ema_loop_prescaled(X, P):
    """X[B,T,D] (already scaled), P[B,T] -> Z[B,T,D];  z_t = (1-p_t) z_{t-1} + x_t."""
    B, T, D = X.shape
    rows = []
    for b in range(B):
        z_prev = torch.zeros(D, dtype=X.dtype)
        steps = []
        for t in range(T):
            z_prev = (1.0 - P[b, t]) * z_prev + X[b, t]
            steps.append(z_prev)
        rows.append(torch.stack(steps))
    return torch.stack(rows)


def north_star_fwd_bwd(x, a, dy=None):
    """x[b,L,h,d], a[b,L,h] or a[h] (torch CPU tensors) -> y, and (dx, da) when dy is given."""
    b, L, h, d = x.shape
    xf = x.detach().permute(0, 2, 1, 3).reshape(b * h, L, d).clone().requires_grad_(dy is not None)
    al = a.detach().clone().requires_grad_(dy is not None)
    a_full = al.view(1, 1, h).expand(b, L, h) if al.dim() == 1 else al
    p = (1.0 - a_full).permute(0, 2, 1).reshape(b * h, L, 1)
    y = ema_loop_pweighted(xf, p)
    unfold = lambda t: t.reshape(b, h, L, d).permute(0, 2, 1, 3).contiguous()
    if dy is None:
        return unfold(y.detach())
    (y * dy.permute(0, 2, 1, 3).reshape(b * h, L, d)).sum().backward()
    return unfold(y.detach()), unfold(xf.grad), al.grad
