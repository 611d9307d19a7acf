"""The C ABI without a GPU: the library loads, exports every symbol include/ema_b200.h declares, and
rejects bad arguments before anything would be launched."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "ema_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ema_b200_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported(ema_lib):
    names = declared_symbols()
    assert len(names) >= 18
    for n in names:
        assert hasattr(ema_lib, n), f"{n} declared in include/ema_b200.h but not exported"


def test_python_binding_covers_the_header(ema_lib):
    assert set(ema_lib._signatures) == set(declared_symbols())


def test_version_and_error_strings(ema_lib):
    assert ema_lib.ema_b200_version() == 100
    for code in range(0, -7, -1):
        assert ema_lib.ema_b200_error_string(code)
    assert b"unknown" in ema_lib.ema_b200_error_string(-99)


def _problem(**kw):
    from ema_b200._lib import Problem
    p = Problem()
    base = dict(b=2, L=256, h=2, d=64, x_sb=256 * 128, x_sl=128, x_sh=64, y_sb=256 * 128, y_sl=128, y_sh=64,
                g_sb=256 * 128, g_sl=128, g_sh=64, a_sb=512, a_sl=2, a_sh=1, dtype=0, decay_mode=0, convention=0,
                chunk=64)
    base.update(kw)
    for k, v in base.items():
        setattr(p, k, v)
    return p


def test_host_only_queries(ema_lib):
    p = _problem()
    assert ema_lib.ema_b200_tile_steps(ctypes.byref(p)) == 128
    assert ema_lib.ema_b200_tile_states_bytes(ctypes.byref(p)) == 4 * 2 * 64 * 4
    assert ema_lib.ema_b200_bwd_workspace_bytes(ctypes.byref(p)) >= 4 * 256 * 4
    bad = _problem(dtype=7)
    assert ema_lib.ema_b200_tile_steps(ctypes.byref(bad)) == 0
    assert ema_lib.ema_b200_tile_states_bytes(ctypes.byref(bad)) == 0


@pytest.mark.parametrize("kw,code", [
    (dict(b=-1), -1), (dict(decay_mode=5), -1), (dict(convention=2), -1), (dict(chunk=-3), -1),
    (dict(dtype=9), -3), (dict(L=1 << 40), -3),
])
def test_bad_problem_is_rejected_before_launch(ema_lib, kw, code):
    p = _problem(**kw)
    one = ctypes.c_void_p(256)
    rc = ema_lib.ema_b200_fwd(ctypes.byref(p), one, one, one, None, None, None, None, None, ctypes.c_float(0), None, 0, None)
    assert rc == code


def test_null_and_misaligned_pointers(ema_lib):
    p = _problem()
    ok = ctypes.c_void_p(256)
    f0 = ctypes.c_float(0)
    assert ema_lib.ema_b200_fwd(None, ok, ok, ok, None, None, None, None, None, f0, None, 0, None) == -1
    assert ema_lib.ema_b200_fwd(ctypes.byref(p), None, ok, ok, None, None, None, None, None, f0, None, 0, None) == -1
    assert ema_lib.ema_b200_fwd(ctypes.byref(p), ok, None, ok, None, None, None, None, None, f0, None, 0, None) == -1
    # no output requested at all
    assert ema_lib.ema_b200_fwd(ctypes.byref(p), ok, ok, None, None, None, None, None, None, f0, None, 0, None) == -1
    # fp32 data at an odd address
    assert ema_lib.ema_b200_fwd(ctypes.byref(p), ctypes.c_void_p(258), ok, ok, None, None, None, None, None, f0, None, 0, None) == -2
    # chunk states without a chunk size
    p0 = _problem(chunk=0)
    assert ema_lib.ema_b200_fwd(ctypes.byref(p0), ok, ok, ok, ok, None, None, None, None, f0, None, 0, None) == -1
    # negative stop threshold
    assert ema_lib.ema_b200_fwd(ctypes.byref(p), ok, ok, ok, None, None, None, None, None, ctypes.c_float(-1), None, 0, None) == -1
    # backward: missing workspace, workspace too small
    assert ema_lib.ema_b200_bwd(ctypes.byref(p), ok, ok, ok, ok, ok, ok, None, None, f0, None, 0, None) == -6
    assert ema_lib.ema_b200_bwd(ctypes.byref(p), ok, ok, ok, ok, ok, ok, None, None, f0, ok, 16, None) == -6
    assert ema_lib.ema_b200_bwd(ctypes.byref(p), ok, ok, None, ok, ok, ok, None, None, f0, ok, 1 << 30, None) == -1
    assert ema_lib.ema_b200_set_path(5) == -1
    # weighted forward: per-step weights need a per-step decay; weights are fp32
    ph = _problem(decay_mode=1)
    assert ema_lib.ema_b200_fwd_weighted(ctypes.byref(ph), ok, ok, ok, None, ok, None, None, None, None, None, f0, None, 0, None) == -3
    assert ema_lib.ema_b200_fwd_weighted(ctypes.byref(p), ok, ok, ctypes.c_void_p(258), None, ok, None, None, None, None, None, f0, None, 0, None) == -2
    assert ema_lib.ema_b200_fwd_weighted(ctypes.byref(p), None, ok, ok, ok, ok, None, None, None, None, None, f0, None, 0, None) == -1


def test_stage_entry_points_reject_bad_sizes(ema_lib):
    ok = ctypes.c_void_p(256)
    assert ema_lib.ema_b200_chunk_cumsum(None, 1, 1, ok, 1, 8, 4, None) == -1
    assert ema_lib.ema_b200_chunk_cumsum(ok, 1, 1, ok, 0, 8, 4, None) == -1
    assert ema_lib.ema_b200_chunk_state(ok, ok, ok, 0, 1, 8, 4, 0, None) == -1
    assert ema_lib.ema_b200_chunk_scan(ok, ok, ok, None, 0, 1, 8, 4, 4, None) == -1
    # without a workspace one thread block walks a whole row: refused beyond 16384 channels
    assert ema_lib.ema_b200_state_passing_bwd(ok, ok, 1, 1, ok, ok, ok, 1, 2, 1 << 20, None, 0, None) == -3
    assert ema_lib.ema_b200_state_passing_bwd_workspace_bytes(2, 3, 1024) == 2 * 3 * 8 * 4
    assert ema_lib.ema_b200_state_passing_bwd_workspace_bytes(2, 3, 1023) == 0
