"""The sequence-parallel algorithm of ema_b200/dist.py run by hand on ONE GPU: the sequence is cut into segments,
every segment is scanned from a zero state, the per-segment records are stacked as the all-gather would deliver
them, folded, and the prefix (forward) / suffix (backward) of each segment is re-scanned in place with
stop_below > 0 into the outputs, saved states, workspace and gradients of the first pass.  Compared with the
sequential definition on the un-split tensors (the C oracle) and with the library's own whole-sequence result.
This covers, without a second GPU, the re-scan path the multi-GPU tests exercise: ema_b200_bwd with stop_below,
dfinal_state and a reused workspace (for bf16 the first pass is made by the tensor-core kernel and the re-scan by the
CUDA-core kernel, which must agree on the layout of the partial sums)."""
import numpy as np
import pytest
import torch

from helpers import check_outputs, make_inputs, oracle_fwd_bwd

pytestmark = pytest.mark.gpu

STOP = 1e-12


def _seq_parallel_by_hand(x, a, dy, n_seg, stop_below=STOP, poison=False):
    from ema_b200 import dist as ed, ops
    b, L, h, d = x.shape
    seg = L // n_seg
    rows = b * h
    per_head = a.dim() == 1
    xs = [x[:, i * seg:(i + 1) * seg] for i in range(n_seg)]
    gs = [dy[:, i * seg:(i + 1) * seg] for i in range(n_seg)]
    as_ = [a if per_head else a[:, i * seg:(i + 1) * seg] for i in range(n_seg)]
    recs = torch.empty((n_seg, rows * d + rows), dtype=torch.float32, device=x.device)
    fw = []
    for i in range(n_seg):
        fin, lds = recs[i, :rows * d].view(b, h, d), recs[i, rows * d:].view(b, h)
        fw.append(ops.ema_fwd(xs[i], as_[i], want_tile_states=True, final_out=fin, log_decay_sum_out=lds))
    # the kernel's fold equals the torch loop of dist.py
    for i in range(n_seg):
        want = ed.fold_carries([r[:rows * d].view(b, h, d) for r in recs], [r[rows * d:].view(b, h) for r in recs], i)
        got = ops.fold_records(recs, i, rows, d).view(b, h, d)
        assert torch.allclose(got, want, rtol=1e-6, atol=1e-6)
    for i in range(1, n_seg):
        carry = ops.fold_records(recs, i, rows, d).view(b, h, d)
        ops.ema_fwd(xs[i], as_[i], init_state=carry, stop_below=stop_below, out=fw[i]["y"],
                    tile_states=fw[i]["tile_states"])
    y = torch.cat([f["y"] for f in fw], dim=1)
    # backward
    brecs = torch.empty_like(recs)
    bw = []
    for i in range(n_seg):
        brecs[i, rows * d:].copy_(recs[i, rows * d:])
        bw.append(ops.ema_bwd(xs[i], as_[i], gs[i], fw[i]["tile_states"], dinit_out=brecs[i, :rows * d].view(b, h, d)))
    first_dx = [r["dx"].clone() for r in bw]
    for i in range(n_seg - 1):
        want = ed.fold_adjoints([r[:rows * d].view(b, h, d) for r in brecs], [r[rows * d:].view(b, h) for r in brecs], i)
        dfinal = ops.fold_records(brecs, i, rows, d, reverse=True).view(b, h, d)
        assert torch.allclose(dfinal, want, rtol=1e-6, atol=1e-6)
        if poison:
            # steps the adjoint can no longer reach must be left alone by the re-scan: mark a prefix of dx
            bw[i]["dx"][:, :128] = 12345.0
        ops.ema_bwd(xs[i], as_[i], gs[i], fw[i]["tile_states"], dfinal_state=dfinal, stop_below=stop_below,
                    dx=bw[i]["dx"], workspace=bw[i]["workspace"], ddecay=bw[i]["ddecay"])
    dx = torch.cat([r["dx"] for r in bw], dim=1)
    da = sum(r["ddecay"] for r in bw) if per_head else torch.cat([r["ddecay"] for r in bw], dim=1)
    return y, dx, da, first_dx, bw


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("per_head", [False, True])
@pytest.mark.parametrize("n_seg", [2, 3])
def test_segments_on_one_gpu_equal_the_whole_sequence(dtype, per_head, n_seg, ema_lib):
    from ema_b200 import ops
    b, h, d = 2, 2, 128
    L = 768 * n_seg
    # long-memory decays: a carry crosses more than one 768-step segment
    x, a, dy, np_in = make_inputs(77 + n_seg, b, L, h, d, lo=3.0, hi=8.0, per_head=per_head, dtype=dtype)
    y, dx, da, _, _ = _seq_parallel_by_hand(x, a, dy, n_seg)
    torch.cuda.synchronize()
    y_ref, dx_ref, da_ref = oracle_fwd_bwd(np_in)
    check_outputs(dtype, y, y_ref, "y")
    check_outputs(dtype, dx, dx_ref, "dx")
    check_outputs(dtype, da, da_ref, "da", grad_of_decay=True)
    # and against the library's own whole-sequence pass
    f = ops.ema_fwd(x, a, want_tile_states=True)
    r = ops.ema_bwd(x, a, dy, f["tile_states"])
    check_outputs(dtype, y, f["y"].float().cpu().numpy(), "y vs whole")
    check_outputs(dtype, dx, r["dx"].float().cpu().numpy(), "dx vs whole")
    assert ema_lib.ema_b200_device_status(1) == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_suffix_rescan_stops_early_and_leaves_the_rest_alone(dtype, ema_lib):
    # short memory (a = 0.5 per head): the adjoint dies within a few tiles, so the re-scan must stop early; the
    # poisoned first tile of dx must survive, and everything else must still be right
    b, h, d, n_seg = 1, 2, 64, 2
    L = 2048
    x, _, dy, np_in = make_inputs(5, b, L, h, d, per_head=True, dtype=dtype)
    a = torch.full((h,), 0.5, dtype=torch.float32, device="cuda")
    y, dx, da, first_dx, bw = _seq_parallel_by_hand(x, a, dy, n_seg, poison=True)
    torch.cuda.synchronize()
    seg = L // n_seg
    assert bool((dx[:, :128] == 12345.0).all()), "the re-scan wrote steps the adjoint cannot reach"
    xn, _, dyn = np_in
    y_ref, dx_ref, da_ref = oracle_fwd_bwd((xn, a.cpu().numpy(), dyn))
    check_outputs(dtype, y, y_ref, "y")
    check_outputs(dtype, dx[:, 128:], dx_ref[:, 128:], "dx past the poisoned tile")
    # the decay gradient was completed from the first pass's partial sums of the untouched tiles
    check_outputs(dtype, da, da_ref, "da", grad_of_decay=True)
    assert ema_lib.ema_b200_device_status(1) == 0
