"""The aggregate schedule of the tensor-core kernels (problems with few work items): a first pass reduces every
128-step tile to its aggregate, and the scan kernels start every piece of a work item from the fold of the
aggregates before (after) it, so that one scan row is spread over many SMs.  Checked against the sequential
definition (the C oracle), against the whole-item schedule of the same kernels, and for independence of where the
pieces are cut (the rows of a problem give the same bits when scanned alone, on a different grid)."""
import numpy as np
import pytest
import torch

from helpers import BF16_REL, assert_close_bf16, assert_close_da_head, make_inputs, oracle_fwd_bwd
from oracle import ema_oracle as eo

pytestmark = pytest.mark.gpu


@pytest.fixture()
def forced(ema_lib):
    """Aggregate schedule for every problem with at least two tiles; restored afterwards."""
    before = ema_lib.ema_b200_set_split(2)
    yield ema_lib
    ema_lib.ema_b200_set_split(before)


def _run(x, a, dy, lib, init=None, dfin=None, chunk=0, prescaled_log=False):
    from ema_b200 import ops
    f = ops.ema_fwd(x, a, init_state=init, want_tile_states=True, want_final=True, chunk=chunk,
                    want_chunk_states=chunk > 0, prescaled_log=prescaled_log)
    sched_f = (lib.ema_b200_last_path(), lib.ema_b200_last_schedule())
    g = ops.ema_bwd(x, a, dy, f["tile_states"], dfinal_state=dfin, want_dinit=True, prescaled_log=prescaled_log)
    sched_b = (lib.ema_b200_last_path(), lib.ema_b200_last_schedule())
    torch.cuda.synchronize()
    return f, g, sched_f, sched_b


# (b, L, h, d): 2, 3 and 7 pieces per item (one tile per thread block), many tiles on a full grid with a ragged end
# and a half-filled channel tile, several rows and heads with two and a half channel tiles
SHAPES = [(1, 256, 1, 128), (1, 384, 1, 64), (1, 896, 1, 128), (1, 128 * 300 + 77, 1, 192), (2, 2048, 3, 320)]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("per_head", [False, True])
def test_pieces_started_from_aggregates_match_the_oracle(shape, per_head, forced):
    lib = forced
    b, L, h, d = shape
    x, a, dy, np_in = make_inputs(300 + L % 97, b, L, h, d, lo=3.0, hi=8.0, per_head=per_head, dtype=torch.bfloat16)
    f, g, sf, sb = _run(x, a, dy, lib)
    assert sf == (1, 2) and sb == (1, 2), "the aggregate schedule did not run"
    y_ref, dx_ref, da_ref = oracle_fwd_bwd(np_in)
    assert_close_bf16(f["y"], y_ref, "y")
    assert_close_bf16(g["dx"], dx_ref, "dx")
    if per_head:
        assert_close_da_head(g["ddecay"], da_ref, np_in, y_ref, dx_ref)
    else:
        assert_close_bf16(g["ddecay"], da_ref, "da")
    # the whole-item schedule of the same kernels
    lib.ema_b200_set_split(0)
    f0, g0, sf0, _ = _run(x, a, dy, lib)
    lib.ema_b200_set_split(2)
    assert sf0 == (1, 0)
    if per_head:   # the decay gradient of the whole-item schedule meets the same bound
        assert_close_da_head(g0["ddecay"], da_ref, np_in, y_ref, dx_ref, "da (whole items)")
    for got, ref, what in ((f["y"], f0["y"], "y"), (g["dx"], g0["dx"], "dx"), (f["final_state"], f0["final_state"], "final"),
                           (f["tile_states"], f0["tile_states"], "tile states"), (g["dinit_state"], g0["dinit_state"], "dinit")):
        ref = ref.float()
        err = float((got.float() - ref).abs().max())
        assert err <= BF16_REL * max(float(ref.abs().max()), 1e-6), f"{what} vs whole items: {err:.3e}"
    assert lib.ema_b200_device_status(1) == 0


@pytest.mark.parametrize("per_head", [False, True])
def test_states_gradients_and_the_log_convention(per_head, forced):
    """Initial state, gradient of the final state, chunk-start states, and the reference's (log a, pre-scaled x)
    convention, all with items cut into pieces."""
    lib = forced
    b, L, h, d = 2, 1000, 2, 256
    x, a, dy, (xn, an, dyn) = make_inputs(9, b, L, h, d, lo=3.0, hi=8.0, per_head=per_head, dtype=torch.bfloat16)
    A = torch.log(a)
    init = torch.randn(b, h, d, device="cuda")
    dfin = torch.randn(b, h, d, device="cuda")
    f, g, sf, sb = _run(x, A, dy, lib, init=init, dfin=dfin, chunk=256, prescaled_log=True)
    assert sf == (1, 2) and sb == (1, 2)
    # oracle with the states: the definition is linear in (x, init), so the initial state enters as a decaying term
    An = np.log(an.astype(np.float64))
    Afull = np.broadcast_to(An.reshape(1, 1, h), (b, L, h)) if per_head else An
    cum = np.cumsum(Afull, axis=1)                                   # log prod_{j<=t} a_j
    y0 = eo.fwd(xn, A.cpu().numpy(), convention=eo.REFERENCE, acc64=True)
    y_ref = y0 + np.exp(cum)[..., None] * init.cpu().numpy()[:, None].astype(np.float64)
    assert_close_bf16(f["y"], y_ref, "y")
    assert_close_bf16(f["final_state"], y_ref[:, -1], "final state")
    want_chunks = np.stack([init.cpu().numpy()] + [y_ref[:, c * 256 - 1] for c in range(1, (L + 255) // 256)], axis=2)
    assert_close_bf16(f["chunk_states"], want_chunks, "chunk-start states")
    # dx: the adjoint of dy plus the decaying adjoint of the final state's gradient
    dx0, _ = eo.bwd(xn, A.cpu().numpy(), dyn, convention=eo.REFERENCE, acc64=True)
    rev = cum[:, -1:, :] - cum                                       # log prod_{t<j<=L-1} a_j
    dx_ref = dx0 + np.exp(rev)[..., None] * dfin.cpu().numpy()[:, None].astype(np.float64)
    assert_close_bf16(g["dx"], dx_ref, "dx")
    dinit_ref = np.exp(Afull[:, 0])[..., None] * dx_ref[:, 0]
    assert_close_bf16(g["dinit_state"], dinit_ref, "dinit")
    assert lib.ema_b200_device_status(1) == 0


@pytest.mark.parametrize("per_head", [False, True])
def test_results_do_not_depend_on_where_the_pieces_are_cut(per_head, forced):
    """The state (adjoint) entering every tile is the same fp32 fold of the aggregates wherever a piece starts, so a
    row scanned alone - another grid, other cuts - gives the same bits as inside the larger problem."""
    lib = forced
    b, L, h, d = 3, 128 * 37, 2, 256
    x, a, dy, _ = make_inputs(55, b, L, h, d, lo=3.0, hi=8.0, per_head=per_head, dtype=torch.bfloat16)
    f, g, sf, sb = _run(x, a, dy, lib)
    assert sf == (1, 2) and sb == (1, 2)
    for bi in range(b):
        a1 = a if per_head else a[bi:bi + 1]
        f1, g1, sf1, _ = _run(x[bi:bi + 1], a1, dy[bi:bi + 1], lib)
        assert sf1 == (1, 2)
        assert torch.equal(f1["y"][0], f["y"][bi]) and torch.equal(g1["dx"][0], g["dx"][bi])
        assert torch.equal(f1["tile_states"], f["tile_states"][bi * h:(bi + 1) * h])
        if not per_head:
            assert torch.equal(g1["ddecay"][0], g["ddecay"][bi])
    assert lib.ema_b200_device_status(1) == 0


def test_few_items_take_the_aggregate_schedule_by_default(ema_lib):
    """4 work items of 16 tiles on a GPU with ~148 SMs: the default setting cuts them into pieces."""
    from ema_b200 import ops
    assert ema_lib.ema_b200_set_split(1) in (0, 1, 2)
    x, a, dy, np_in = make_inputs(12, 1, 2048, 2, 256, per_head=True, dtype=torch.bfloat16)
    f, g, sf, sb = _run(x, a, dy, ema_lib)
    assert sf == (1, 2) and sb == (1, 2)
    y_ref, dx_ref, da_ref = oracle_fwd_bwd(np_in)
    assert_close_bf16(f["y"], y_ref, "y")
    assert_close_bf16(g["dx"], dx_ref, "dx")
    assert_close_da_head(g["ddecay"], da_ref, np_in, y_ref, dx_ref)
    # many items: the schedule is not used (256 items), nor when the summed log decay is asked for
    x2, a2, _, _ = make_inputs(13, 16, 512, 2, 1024, per_head=True, dtype=torch.bfloat16)
    ops.ema_fwd(x2, a2)
    assert ema_lib.ema_b200_last_schedule() in (0, 1)
    ops.ema_fwd(x, a, want_log_decay_sum=True)
    assert ema_lib.ema_b200_last_schedule() == 0
    assert ema_lib.ema_b200_device_status(1) == 0
