"""The binding stubs a maintainer of the reference would add (triton-kernels_b200/examples/reference_binding_stub.py, the
file the integration notes quote) are imported as they stand and their results compared with the package's own entry
points."""
import importlib.util
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _stub_namespace(ema_lib):
    path = os.path.join(ROOT, "triton-kernels_b200", "examples", "reference_binding_stub.py")
    os.environ.setdefault("EMA_B200_LIB", ema_lib._name)
    spec = importlib.util.spec_from_file_location("reference_binding_stub", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return vars(mod)


def test_forward_stub(ema_lib):
    from ema_b200 import ops
    ns = _stub_namespace(ema_lib)
    B, L, T, Q = 3, 500, 192, 64
    g = torch.Generator(device="cuda").manual_seed(5)
    A = -0.1 * torch.rand((B, L), generator=g, device="cuda")
    X = torch.randn((B, L, T), generator=g, device="cuda")
    out, states, final = ns["ema_matmul_scan_combined_fwd"](A, X, Q)
    ref = ops.ema_fwd(X.view(B, L, 1, T), A.view(B, L, 1), prescaled_log=True, chunk=Q, want_chunk_states=True,
                      want_final=True)
    assert torch.equal(out, ref["y"].view(B, L, T))
    assert torch.equal(states, ref["chunk_states"].view(B, -1, T))
    assert torch.equal(final, ref["final_state"].view(B, T))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_weighted_forward_stub(dtype, ema_lib):
    from kernels.ema_combined import ema_chunk_scan_combined
    ns = _stub_namespace(ema_lib)
    b, l, h, d = 2, 300, 2, 128
    g = torch.Generator(device="cuda").manual_seed(6)
    x = torch.randn((b, l, h, d), generator=g, device="cuda").to(dtype)
    dt = 0.01 + 0.2 * torch.rand((b, l, h), generator=g, device="cuda")
    A = -torch.rand((h,), generator=g, device="cuda")
    Bw = torch.rand((b, l, h), generator=g, device="cuda")
    Cw = torch.randn((b, l, h), generator=g, device="cuda")
    out = ns["ema_chunk_scan_combined_inference"](x, dt, A, Bw, Cw)
    with torch.no_grad():
        ref = ema_chunk_scan_combined(x, dt, A, Bw.unsqueeze(-1), Cw.unsqueeze(-1), chunk_size=64)
    assert torch.equal(out, ref)
