"""The optional per-call trace (EMA_B200_TRACE=<file>, EMA_B200_NVTX=1): one JSON line per library call with the shape,
the kernel family and schedule that ran, and the time between two CUDA events around the call."""
import json

import pytest
import torch

from helpers import make_inputs

pytestmark = pytest.mark.gpu


def test_trace_file_gets_one_record_per_call(tmp_path, monkeypatch, ema_lib):
    from ema_b200 import ops
    path = tmp_path / "trace.jsonl"
    monkeypatch.setenv("EMA_B200_TRACE", str(path))
    monkeypatch.setenv("EMA_B200_NVTX", "1")
    x, a, dy, _ = make_inputs(1, 2, 600, 2, 128, per_head=True, dtype=torch.bfloat16)
    f = ops.ema_fwd(x, a, want_tile_states=True)
    ops.ema_bwd(x, a, dy, f["tile_states"])
    monkeypatch.delenv("EMA_B200_TRACE")
    ops.ema_fwd(x, a)                      # not traced any more
    recs = [json.loads(line) for line in path.read_text().splitlines()]
    assert [r["op"] for r in recs] == ["ema_fwd", "ema_bwd"]
    for r in recs:
        assert r["shape"] == [2, 600, 2, 128] and r["dtype"] == "bfloat16" and r["decay"] == "per_head"
        assert r["path"] == 1 and r["ms"] > 0 and r["algorithmic_GBps"] > 0 and r["tokens_per_s"] > 0
