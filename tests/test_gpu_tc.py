"""The tensor-core (tcgen05 + TMA) path for bf16 problems: against the CPU oracle, against the
CUDA-core path on the same inputs, and the device status word (no bounded wait may run out)."""
import numpy as np
import pytest
import torch

from helpers import assert_close_bf16, make_inputs, oracle_fwd_bwd
from oracle import ema_oracle as eo

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _lib(ema_lib):
    assert torch.cuda.is_available()
    ema_lib.ema_b200_set_path(0)
    yield ema_lib
    ema_lib.ema_b200_set_path(0)
    assert ema_lib.ema_b200_device_status(1) == 0, "a device-side wait timed out during these tests"


def _E():
    import ema_b200
    return ema_b200


TC_SHAPES = [
    (1, 128, 1, 64),     # exactly one tile, one item
    (1, 40, 1, 8),       # a fraction of a tile, d far below the 64-channel box
    (2, 129, 2, 24),     # ragged by one step, d not a multiple of 64
    (1, 640, 3, 128),    # several tiles, several channel tiles, three heads
    (5, 300, 2, 1024),   # 160 work items: every CTA walks two of them
    (2, 1111, 4, 256),
]


@pytest.mark.parametrize("shape", TC_SHAPES)
@pytest.mark.parametrize("per_head", [False, True])
def test_tc_forward_matches_oracle(shape, per_head, _lib):
    b, L, h, d = shape
    x, a, dy, np_in = make_inputs(500 + L + d, b, L, h, d, per_head=per_head, dtype=torch.bfloat16)
    y_ref = eo.fwd(np_in[0], np_in[1], acc64=True)
    r = _E().ema_fwd(x, a, want_final=True)
    assert_close_bf16(r["y"], y_ref, "y")
    assert_close_bf16(r["final_state"], np.ascontiguousarray(y_ref[:, -1]), "final state", rel=1e-2)
    assert _lib.ema_b200_device_status(1) == 0


@pytest.mark.parametrize("per_head", [False, True])
def test_tc_equals_fma_path(per_head, _lib):
    """Same inputs through both kernel families: bf16 outputs agree to bf16 rounding, fp32 side
    outputs (saved states, final state, log-decay sum) to 5e-3 of their scale: the tensor-core path
    rounds the decay matrix to bf16 (8 mantissa bits), the CUDA-core path keeps decays in fp32."""
    E = _E()
    b, L, h, d = 2, 700, 2, 192
    x, a, _, _ = make_inputs(77, b, L, h, d, per_head=per_head, dtype=torch.bfloat16)
    init = torch.randn(b, h, d, device="cuda")
    kw = dict(chunk=100, want_chunk_states=True, want_tile_states=True, want_final=True,
              want_log_decay_sum=True, init_state=init)
    _lib.ema_b200_set_path(1)
    f = E.ema_fwd(x, a, **kw)
    _lib.ema_b200_set_path(0)
    t = E.ema_fwd(x, a, **kw)
    for key, rel in (("y", 1.6e-2), ("chunk_states", 5e-3), ("tile_states", 5e-3), ("final_state", 5e-3),
                     ("log_decay_sum", 1e-4)):
        ref = f[key].float().cpu().numpy()
        assert_close_bf16(t[key], ref, key, rel=rel)
    assert _lib.ema_b200_device_status(1) == 0


def test_tc_prescaled_log_convention(_lib):
    E = _E()
    b, L, h, d = 2, 300, 1, 64
    rs = np.random.RandomState(5)
    A = (-0.05 * rs.random_sample((b, L, h))).astype(np.float32)
    U = torch.tensor(rs.standard_normal((b, L, h, d)).astype(np.float32)).to(torch.bfloat16)
    y_ref = eo.fwd(U.float().numpy(), A, convention=eo.REFERENCE, acc64=True)
    r = E.ema_fwd(U.cuda(), torch.tensor(A).cuda(), prescaled_log=True)
    assert_close_bf16(r["y"], y_ref, "y")


def test_tc_forward_feeds_backward(_lib):
    """States saved by the tensor-core forward drive the backward (dx, da against the oracle)."""
    b, L, h, d = 2, 520, 2, 128
    for per_head in (False, True):
        x, a, dy, np_in = make_inputs(91, b, L, h, d, per_head=per_head, dtype=torch.bfloat16)
        y_ref, dx_ref, da_ref = oracle_fwd_bwd(np_in)
        x.requires_grad_(True)
        a.requires_grad_(True)
        y = _E().ema(x, a)
        y.backward(dy)
        assert_close_bf16(y, y_ref, "y")
        assert_close_bf16(x.grad, dx_ref, "dx")
        assert_close_bf16(a.grad, da_ref, "da")
    assert _lib.ema_b200_device_status(1) == 0


def test_tc_strided_views(_lib):
    """[b,h,L,d] storage viewed as [b,L,h,d]: the tensor map carries the strides, no copy is made."""
    E = _E()
    b, L, h, d = 2, 260, 2, 64
    xs = torch.randn(b, h, L, d, device="cuda").to(torch.bfloat16).permute(0, 2, 1, 3)
    a = torch.sigmoid(2 + 4 * torch.rand(b, L, h, device="cuda"))
    y1 = E.ema_fwd(xs, a)["y"]
    y2 = E.ema_fwd(xs.contiguous(), a)["y"]
    assert torch.equal(y1, y2)


@pytest.mark.parametrize("shape", TC_SHAPES)
@pytest.mark.parametrize("per_head", [False, True])
def test_tc_backward_matches_oracle(shape, per_head, _lib):
    b, L, h, d = shape
    x, a, dy, np_in = make_inputs(900 + L + d, b, L, h, d, per_head=per_head, dtype=torch.bfloat16)
    _, dx_ref, da_ref = oracle_fwd_bwd(np_in)
    E = _E()
    f = E.ema_fwd(x, a, want_tile_states=True)
    g = E.ema_bwd(x, a, dy, f["tile_states"])
    assert_close_bf16(g["dx"], dx_ref, "dx")
    assert_close_bf16(g["ddecay"], da_ref, "da")
    assert _lib.ema_b200_device_status(1) == 0


@pytest.mark.parametrize("per_head", [False, True])
@pytest.mark.parametrize("prescaled", [False, True])
def test_tc_backward_equals_fma_path(per_head, prescaled, _lib):
    """Both kernel families on the same inputs and the same saved states, including the adjoint entering
    from the right (dfinal) and the one leaving on the left (dinit)."""
    E = _E()
    b, L, h, d = 2, 450, 2, 192
    x, a, dy, _ = make_inputs(78, b, L, h, d, per_head=per_head, dtype=torch.bfloat16)
    if prescaled:
        a = torch.log(a)
    dfin = torch.randn(b, h, d, device="cuda")
    _lib.ema_b200_set_path(1)
    f = E.ema_fwd(x, a, want_tile_states=True, prescaled_log=prescaled)
    gf = E.ema_bwd(x, a, dy, f["tile_states"], dfinal_state=dfin, want_dinit=True, prescaled_log=prescaled)
    _lib.ema_b200_set_path(0)
    gt = E.ema_bwd(x, a, dy, f["tile_states"], dfinal_state=dfin, want_dinit=True, prescaled_log=prescaled)
    for key, rel in (("dx", 1.6e-2), ("ddecay", 5e-3), ("dinit_state", 5e-3)):
        assert_close_bf16(gt[key], gf[key].float().cpu().numpy(), key, rel=rel)
    assert _lib.ema_b200_device_status(1) == 0


SPLIT_SHAPES = [
    (10, 640, 2, 1024),    # 160 items of 5 tiles on 148 SMs
    (19, 300, 1, 1024),    # 152 items of 3 tiles, ragged last tile
    (3, 2000, 7, 1000),    # 168 items of 16 tiles, d not a multiple of 128
    (19, 300, 8, 1024),    # per-step decay: 608 two-tile items cut over the SMs; per-head: 1216 items
    (37, 260, 1, 640),     # 185 items per-head; five channel tiles, i.e. an odd one left over when they are paired
]


@pytest.mark.parametrize("shape", SPLIT_SHAPES)
@pytest.mark.parametrize("per_head", [False, True])
def test_items_cut_across_thread_blocks_give_identical_results(shape, per_head, _lib):
    """When the work items do not divide evenly among the SMs the kernels cut some of them across thread blocks
    and hand the carries through global memory: same arithmetic per tile, so bit-identical outputs."""
    if torch.cuda.get_device_properties(0).multi_processor_count != 148:
        pytest.skip("shapes chosen for 148 SMs")
    E = _E()
    b, L, h, d = shape
    x, a, dy, np_in = make_inputs(77, b, L, h, d, per_head=per_head, dtype=torch.bfloat16)
    init = torch.randn(b, h, d, device="cuda")
    dfin = torch.randn(b, h, d, device="cuda")
    res = []
    for split in (1, 0):
        _lib.ema_b200_set_split(split)
        f = E.ops.ema_fwd(x, a, init_state=init, want_tile_states=True, want_final=True, chunk=128, want_chunk_states=True)
        g = E.ops.ema_bwd(x, a, dy, f["tile_states"], dfinal_state=dfin, want_dinit=True)
        torch.cuda.synchronize()
        assert _lib.ema_b200_last_path() == 1
        res.append((f["y"], f["final_state"], f["chunk_states"], f["tile_states"], g["dx"], g["ddecay"], g["dinit_state"]))
    _lib.ema_b200_set_split(1)
    for got, ref, what in zip(res[0], res[1], ("y", "final", "chunk_states", "tile_states", "dx", "da", "dinit")):
        assert torch.equal(got, ref), what
    assert _lib.ema_b200_device_status(0) == 0
    # and the plain problem (no initial state) against the oracle
    f = E.ops.ema_fwd(x, a, want_tile_states=True)
    g = E.ops.ema_bwd(x, a, dy, f["tile_states"])
    y_ref, dx_ref, da_ref = oracle_fwd_bwd(np_in)
    assert_close_bf16(f["y"], y_ref, "y")
    assert_close_bf16(g["dx"], dx_ref, "dx")
    assert_close_bf16(g["ddecay"], da_ref, "da")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_decays_from_zero_to_one(dtype, _lib):
    """Per-step decays over the whole range, exact 0 and exact 1 included: the log-domain matrices of the tensor-core
    kernels and the plain recurrence of the CUDA-core kernels must both stay finite and agree with the oracle."""
    E = _E()
    b, L, h, d = 2, 700, 2, 128
    x, a, dy, _ = make_inputs(31, b, L, h, d, lo=-20.0, hi=12.0, per_head=False, dtype=dtype)
    g = torch.Generator().manual_seed(5)
    pick = torch.randint(0, 12, a.shape, generator=g).cuda()
    special = torch.tensor([0.0, 1e-30, 1e-6, 1.0], device="cuda")
    a = torch.where(pick < 4, special[pick.clamp(max=3)], a).contiguous()
    np_in = (x.float().cpu().numpy(), a.cpu().numpy(), dy.float().cpu().numpy())
    f = E.ops.ema_fwd(x, a, want_tile_states=True)
    r = E.ops.ema_bwd(x, a, dy, f["tile_states"])
    torch.cuda.synchronize()
    assert _lib.ema_b200_last_path() == (1 if dtype == torch.bfloat16 else 2)   # tensor cores | CUDA cores fed by TMA
    y_ref, dx_ref, da_ref = oracle_fwd_bwd(np_in)
    for got in (f["y"], r["dx"], r["ddecay"]):
        assert bool(torch.isfinite(got.float()).all())
    if dtype == torch.bfloat16:
        assert_close_bf16(f["y"], y_ref, "y")
        assert_close_bf16(r["dx"], dx_ref, "dx")
        assert_close_bf16(r["ddecay"], da_ref, "da")
    else:
        assert np.abs(f["y"].cpu().numpy() - y_ref).max() <= 1e-4
        assert np.abs(r["dx"].cpu().numpy() - dx_ref).max() <= 1e-4
        assert np.abs(r["ddecay"].cpu().numpy() - da_ref).max() <= 1e-4 + 2e-5 * np.abs(da_ref).max()


def test_many_restarts_inside_a_tile(_lib):
    """Short packed sequences: a decay of exactly 0 every third step (the state restarts there) and slow decays in
    between.  The prefix sums of the log decays inside a tile cross dozens of such steps and must stay precise."""
    E = _E()
    b, L, h, d = 2, 520, 2, 256
    x, a, dy, _ = make_inputs(47, b, L, h, d, lo=3.0, hi=8.0, per_head=False, dtype=torch.bfloat16)
    a = a.clone()
    a[:, ::3] = 0.0
    np_in = (x.float().cpu().numpy(), a.cpu().numpy(), dy.float().cpu().numpy())
    f = E.ops.ema_fwd(x, a, want_tile_states=True)
    r = E.ops.ema_bwd(x, a, dy, f["tile_states"])
    torch.cuda.synchronize()
    assert _lib.ema_b200_last_path() == 1
    y_ref, dx_ref, da_ref = oracle_fwd_bwd(np_in)
    assert_close_bf16(f["y"], y_ref, "y")
    assert_close_bf16(r["dx"], dx_ref, "dx")
    assert_close_bf16(r["ddecay"], da_ref, "da")
    # the steps between restarts carry small weights (1 - a down to 3e-4): check them on their own scale
    mid = np.ones(L, dtype=bool)
    mid[::3] = False
    got, ref = r["dx"].float().cpu().numpy()[:, mid], dx_ref[:, mid]
    assert np.abs(got - ref).max() <= 2e-2 * np.abs(ref).max()


def test_calls_can_be_captured_in_cuda_graphs(_lib):
    if _lib.ema_b200_bounds_checked():
        pytest.skip("the bounds-checking build rewrites its table from host memory before every launch: not capturable")
    """With caller-provided buffers a forward and a backward call only queue stream work (kernels and two small
    memsets), so they capture into CUDA graphs; a replay must reproduce the eager results bit for bit."""
    E = _E()
    b, L, h, d = 10, 640, 2, 1024   # enough items for the tile-range schedule, whose counters a memset node clears
    x, a, dy, _ = make_inputs(91, b, L, h, d, per_head=True, dtype=torch.bfloat16)
    y, dx, da = torch.empty_like(x), torch.empty_like(x), torch.empty_like(a)
    f = E.ops.ema_fwd(x, a, out=y, want_tile_states=True)
    ts, fws = f["tile_states"], f["fwd_workspace"]
    ws = E.ops.ema_bwd(x, a, dy, ts, dx=dx, ddecay=da)["workspace"]
    torch.cuda.synchronize()
    ref = (y.clone(), dx.clone(), da.clone())
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):   # warm-up on a side stream, as graph capture wants
        E.ops.ema_fwd(x, a, out=y, tile_states=ts, workspace=fws)
        E.ops.ema_bwd(x, a, dy, ts, dx=dx, ddecay=da, workspace=ws)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        E.ops.ema_fwd(x, a, out=y, tile_states=ts, workspace=fws)
        E.ops.ema_bwd(x, a, dy, ts, dx=dx, ddecay=da, workspace=ws)
    for _ in range(2):
        y.zero_(); dx.zero_(); da.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(y, ref[0]) and torch.equal(dx, ref[1]) and torch.equal(da, ref[2])
    assert _lib.ema_b200_device_status(0) == 0
