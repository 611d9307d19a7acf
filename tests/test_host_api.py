"""Host-side behaviour that needs no GPU: the drop-ins keep the reference's signatures, refuse CPU
tensors (there is no CPU path), and validate shapes like the reference."""
import inspect

import pytest
import torch

import ema_b200
from ema_b200 import dist as ema_dist

# parameter lists read off the reference project (file:line of each `def`)
REFERENCE_SIGNATURES = {
    ("kernels.ema", "ema_scan_combined"): ["x", "p"],                                      # kernels/ema.py:370
    ("kernels.ema_kernels.ema_cumsum", "ema_chunk_cumsum_fwd"): ["A", "chunk_size"],        # ema_cumsum.py:66
    ("kernels.ema_kernels.ema_state_fwd", "_ema_chunk_state_fwd"):
        ["x", "A_cumsum", "seq_idx", "states", "states_in_fp32"],                          # ema_state_fwd.py:130
    ("kernels.ema_kernels.ema_state_pass", "_ema_state_passing_fwd"):
        ["states", "A_cs_last", "initial_states", "chunk_size", "out_dtype"],              # ema_state_pass.py:125
    ("kernels.ema_kernels.ema_scan_fwd", "_ema_scan_fwd"): ["x", "A_cumsum", "states"],     # ema_scan_fwd.py:161
    ("kernels.ema_kernels.ema_combined_fwd", "_ema_matmul_scan_combined_fwd"):
        ["A_ema", "X_ema", "chunk_size", "dtype"],                                         # ema_combined_fwd.py:12
    ("kernels.ema_kernels.ema_combined_fwd", "ema_matmul_scan_combined"): ["A_ema", "X_ema", "chunk_size"],  # :75
    ("kernels.ema_kernels_bwd.ema_scan_bwd", "_ema_chunk_scan_bwd_dstates"):
        ["dA_cumsum", "dout", "seq_idx", "dtype"],                                         # ema_scan_bwd.py:132
    ("kernels.ema_kernels_bwd.ema_state_passing_bwd_dstates", "_ema_state_passing_bwd"):
        ["states", "dA_chunk_cumsum", "dout", "dfinal_states", "seq_idx", "has_initial_states", "dstates_dtype",
         "states_dtype", "chunk_size"],                                                    # ..._bwd_dstates.py:103
    ("kernels.ema_kernels_bwd.ema_chunk_scan_chunk_state_bwd_dx", "_chunk_scan_chunk_state_bwd_dx"):
        ["x", "dA_cumsum", "dout", "dstates", "D", "seq_idx", "dx"],                       # ..._bwd_dx.py:208
    ("kernels.ema_kernels_bwd.ema_chunk_state_bwd_db", "_ema_chunk_state_bwd_db"):
        ["x", "dA_cumsum", "dstates", "seq_idx", "B", "ngroups", "raw_scale_gradient"],    # ..._bwd_db.py:122
    ("kernels.ema_kernels_bwd.ema_chunk_scan_bwd_dc", "_ema_chunk_scan_bwd_dC"):
        ["prev_states", "dA_cumsum", "dout", "seq_idx", "C", "ngroups"],                   # ..._bwd_dc.py:115
    ("kernels.ema_kernels_bwd.ema_scan_da", "_ema_chunk_scan_bwd_ddAcs_stable"): ["x", "dA_cumsum", "dout"],  # :113
    ("kernels.ema_kernels_bwd.ema_combined_bwd", "_ema_chunk_scan_combined_bwd"):
        ["dout", "x", "A", "chunk_size", "dt_limit", "recompute_output"],                  # ema_combined_bwd.py:13
}


@pytest.mark.parametrize("key", sorted(REFERENCE_SIGNATURES))
def test_drop_in_signatures_match_the_reference(key):
    mod = __import__(key[0], fromlist=[key[1]])
    fn = getattr(mod, key[1])
    assert list(inspect.signature(fn).parameters) == REFERENCE_SIGNATURES[key]


def test_autograd_classes_exist_with_reference_names():
    from kernels.ema import EMAChunkScanCombinedFn
    from kernels.ema_kernels.ema_combined_fwd import EMAMatmulCombinedFn
    assert issubclass(EMAChunkScanCombinedFn, torch.autograd.Function)
    assert issubclass(EMAMatmulCombinedFn, torch.autograd.Function)


def test_no_cpu_path():
    x = torch.zeros(1, 8, 1, 8)
    a = torch.full((1, 8, 1), 0.9)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        ema_b200.ema(x, a)
    from kernels.ema_kernels.ema_cumsum import ema_chunk_cumsum_fwd
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        ema_chunk_cumsum_fwd(torch.zeros(2, 16), 8)
    from kernels.ema_kernels.ema_combined_fwd import ema_matmul_scan_combined
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        ema_matmul_scan_combined(torch.zeros(2, 16), torch.zeros(2, 16, 4), 8)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from ema_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setenv("EMA_B200_LIB", str(tmp_path / "nope.so"))
    with pytest.raises(ema_b200.EmaB200Error, match="not found"):
        _lib.lib()
    monkeypatch.delenv("EMA_B200_LIB")
    monkeypatch.setattr(_lib, "_lib", None)
    assert _lib.lib().ema_b200_version() == 100


def test_shape_validation():
    from ema_b200 import ops
    with pytest.raises(ValueError):
        ops._check_inputs(torch.zeros(2, 3, 4), torch.zeros(2))
    with pytest.raises(ValueError):
        ops._check_inputs(torch.zeros(2, 3, 4, 5), torch.zeros(3))
    with pytest.raises(ValueError):
        ops._check_inputs(torch.zeros(2, 3, 4, 5), torch.zeros(2, 3, 5))
    x, a = ops._check_inputs(torch.zeros(2, 3, 4, 5).transpose(2, 3), torch.zeros(5, dtype=torch.float64))
    assert x.stride(-1) == 1 and a.dtype == torch.float32


def test_reference_asserts_are_kept():
    from kernels.ema import ema_scan_combined
    from kernels.ema_kernels.ema_state_pass import _ema_state_passing_fwd
    with pytest.raises(AssertionError):
        ema_scan_combined(torch.zeros(2, 8, 4).transpose(1, 2), torch.zeros(2, 4, 1))
    with pytest.raises(NotImplementedError):
        _ema_state_passing_fwd(torch.zeros(2, 3, 4), torch.zeros(2, 3), initial_states=torch.zeros(2, 4))
    with pytest.raises(AssertionError):
        _ema_state_passing_fwd(torch.zeros(2, 3, 4), torch.zeros(2, 4))


@pytest.mark.parametrize("b,h,world", [(16, 2, 8), (4, 8, 8), (8, 4, 2), (3, 2, 2), (1, 8, 4), (16, 2, 1)])
def test_row_shard_plan_covers_every_row_once(b, h, world):
    plan = ema_dist.plan_row_shards(b, h, world)
    assert len(plan) == world
    seen = set()
    for (b0, b1, h0, h1) in plan:
        for bi in range(b0, b1):
            for hi in range(h0, h1):
                assert (bi, hi) not in seen
                seen.add((bi, hi))
    assert len(seen) == b * h
    sizes = [(b1 - b0) * (h1 - h0) for (b0, b1, h0, h1) in plan]
    if (b * h) % world == 0 and (b % world == 0 or (world % b == 0 and h % (world // b) == 0)):
        assert len(set(sizes)) == 1
