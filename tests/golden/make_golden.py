"""Regenerate the golden fixtures in this directory from the reference checkout.

Run once, in a container that has the reference project checked out (CPU only):

    python tests/golden/make_golden.py --ref /path/to/triton-kernels

Two sources of truth are recorded, both executed from the reference's own files:

* the sequential PyTorch EMA loops (kernels/tests/ema/test_ema_scan_fwd.py:25-37, p-weighted;
  kernels/tests/ema_bwd/_ema_full_bwd.py:24-34, pre-scaled) and autograd through them, and
* the reference's Triton stage kernels executed by Triton's CPU interpreter
  (TRITON_INTERPRET=1), with two harness-side shims that leave the reference untouched:
  `torch.cuda.device` becomes a null context for CPU tensors, and every autotuned kernel is
  pinned to one configuration (the autotuner cannot benchmark without a GPU).  The reverse
  state-passing kernel is pinned to BLOCK_SIZE=64, the block size its host wrapper sizes the
  partial-sum buffer for (kernels/ema_kernels_bwd/ema_state_passing_bwd_dstates.py:134-142).

* the heads-style entry point ema_chunk_scan_combined (kernels/ema_combined.py:100, forward :12-57) for state
  size 1, again through the interpreted Triton kernels, each autotuner pinned to its first configuration.  Its
  cumulative-sum kernel hard-codes dA = -dt (kernels/ema_chunk_state.py:95), so only A = -1 is comparable with
  the sequential definition; the fixtures record that in `meta_A_is_minus_one`.

Inputs come from numpy's frozen RandomState streams (golden_inputs.py); the north-star fixtures
store only a and the outputs, and the tests rebuild x and dy from the recorded seed.
"""
import argparse
import contextlib
import os
import sys

import numpy as np


sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from golden_inputs import gen_inputs  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("EMA_REFERENCE_CHECKOUT"), required=os.environ.get("EMA_REFERENCE_CHECKOUT") is None,
                    help="path of a checkout of the reference project (kartiksrinivas007/triton-kernels)")
    ap.add_argument("--out", default=os.path.dirname(os.path.abspath(__file__)))
    ap.add_argument("--only", default=None, choices=[None, "heads_varlen"], help="record only this group of fixtures")
    args = ap.parse_args()

    os.environ["TRITON_INTERPRET"] = "1"
    sys.path.insert(0, args.ref)
    import torch
    import triton

    torch.cuda.device = lambda index: contextlib.nullcontext()
    torch.set_num_threads(4)

    from kernels.tests.ema.test_ema_scan_fwd import ema_loop as ema_loop_pweighted
    from kernels.tests.ema_bwd._ema_full_bwd import ema_loop as ema_loop_prescaled
    from kernels.ema_kernels import ema_cumsum, ema_state_fwd, ema_state_pass, ema_scan_fwd
    from kernels.ema_kernels_bwd import (ema_chunk_scan_bwd_dc, ema_chunk_scan_chunk_state_bwd_dx,
                                         ema_chunk_state_bwd_db, ema_scan_bwd, ema_scan_da,
                                         ema_state_passing_bwd_dstates)
    from kernels.ema_kernels_bwd.ema_combined_bwd import _ema_chunk_scan_combined_bwd
    from kernels.ema_kernels.ema_combined_fwd import _ema_matmul_scan_combined_fwd

    for mod, name in [(ema_cumsum, "ema_chunk_cumsum_fwd_kernel"),
                      (ema_state_fwd, "_ema_chunk_state_fwd_kernel"),
                      (ema_state_pass, "_ema_state_passing_fwd_kernel"),
                      (ema_scan_fwd, "_ema_scan_fwd_kernel"),
                      (ema_scan_bwd, "_ema_chunk_scan_bwd_dstates_kernel"),
                      (ema_chunk_scan_chunk_state_bwd_dx, "_chunk_scan_chunk_state_bwd_dx_kernel"),
                      (ema_chunk_state_bwd_db, "_ema_chunk_state_bwd_db_kernel"),
                      (ema_chunk_scan_bwd_dc, "_ema_chunk_scan_bwd_dc_kernel"),
                      (ema_scan_da, "_ema_chunk_scan_bwd_ddAcs_stable_kernel")]:
        kern = getattr(mod, name)
        kern.configs = kern.configs[:1]
    spb = ema_state_passing_bwd_dstates._ema_state_passing_bwd_kernel
    spb.configs = [triton.Config({"BLOCK_SIZE": 64})]

    def fold(t4):  # [b,L,h,d] -> [b*h, L, d]
        b, L, h, d = t4.shape
        return np.ascontiguousarray(t4.transpose(0, 2, 1, 3)).reshape(b * h, L, d)

    def north_star_case(name, seed, b, L, h, d, lo, hi, per_head):
        """y, dx, da from the reference's p-weighted sequential loop and autograd through it."""
        x, a, dy = gen_inputs(seed, b, L, h, d, lo, hi, per_head)
        xt = torch.tensor(fold(x), requires_grad=True)
        at = torch.tensor(a, requires_grad=True)
        a_full = at.view(1, 1, h).expand(b, L, h) if per_head else at
        p = (1.0 - a_full).permute(0, 2, 1).reshape(b * h, L, 1)
        y = ema_loop_pweighted(xt, p)
        (y * torch.tensor(fold(dy))).sum().backward()
        unfold = lambda t: t.detach().numpy().reshape(b, h, L, d).transpose(0, 2, 1, 3)
        np.savez(os.path.join(args.out, name + ".npz"), a=a,
                 y=np.ascontiguousarray(unfold(y)), dx=np.ascontiguousarray(unfold(xt.grad)),
                 da=at.grad.numpy(), meta=np.array([seed, b, L, h, d, int(per_head)]),
                 lohi=np.array([lo, hi]))
        print(name, "done", float(y.detach().abs().max()))

    def stage_case(name, seed, B, L, T, Q, scale):
        """Every intermediate of the reference's chunked pipeline (interpreted Triton kernels),
        plus out/dX/dA from its pre-scaled sequential loop and autograd."""
        rs = np.random.RandomState(seed)
        A = (-scale * rs.random_sample((B, L))).astype(np.float32)
        X = rs.standard_normal((B, L, T)).astype(np.float32)
        dout = rs.standard_normal((B, L, T)).astype(np.float32)
        At = torch.tensor(A, requires_grad=True)
        Xt = torch.tensor(X, requires_grad=True)
        P = 1 - torch.exp(At)
        out = ema_loop_prescaled(Xt, P)
        (out * torch.tensor(dout)).sum().backward()
        rec = dict(A=A, X=X, dout=dout, loop_out=out.detach().numpy(), loop_dX=Xt.grad.numpy(),
                   loop_dA=At.grad.numpy(), meta=np.array([seed, B, L, T, Q]))
        with torch.no_grad():
            A_, X_, d_ = torch.tensor(A), torch.tensor(X), torch.tensor(dout)
            o, cs, h, fin = _ema_matmul_scan_combined_fwd(A_, X_, Q)
            S = ema_state_fwd._ema_chunk_state_fwd(X_, cs)
            dh_scan = ema_scan_bwd._ema_chunk_scan_bwd_dstates(cs, d_, dtype=torch.float32)
            dS, ddA_last, _ = ema_state_passing_bwd_dstates._ema_state_passing_bwd(
                h, cs[..., -1], dh_scan, chunk_size=Q)
            dx = ema_chunk_scan_chunk_state_bwd_dx._chunk_scan_chunk_state_bwd_dx(X_, cs, d_, dS)
            db_raw = ema_chunk_state_bwd_db._ema_chunk_state_bwd_db(X_, cs, dS, raw_scale_gradient=True)
            db = ema_chunk_state_bwd_db._ema_chunk_state_bwd_db(X_, cs, dS)
            dc = ema_chunk_scan_bwd_dc._ema_chunk_scan_bwd_dC(h, cs, d_)
            dacs = ema_scan_da._ema_chunk_scan_bwd_ddAcs_stable(X_, cs, d_)
            cdx, cddA, cout = _ema_chunk_scan_combined_bwd(d_, X_, A_, Q, recompute_output=True)
        rec.update(out=o.numpy(), cs=cs.numpy(), chunk_start_states=h.numpy(), final=fin.numpy(),
                   S=S.numpy(), dh_scan=dh_scan.numpy(), dS=dS.numpy(), ddA_last=ddA_last.numpy(),
                   dx=dx.numpy(), db_raw=db_raw.numpy(), db=db.numpy(), dc=dc.numpy(),
                   dacs=dacs.numpy(), comb_dx=cdx.numpy(), comb_ddA=cddA.numpy(), comb_out=cout.numpy())
        np.savez(os.path.join(args.out, name + ".npz"), **rec)
        L_pad = cddA.shape[1] * cddA.shape[2]
        err = np.abs(cddA.numpy().reshape(B, L_pad)[:, :L] - rec["loop_dA"]).max()
        print(name, "done; combined ddA vs autograd:", err,
              "dx:", np.abs(cdx.numpy() - rec["loop_dX"]).max(),
              "out:", np.abs(o.numpy() - rec["loop_out"]).max())

    def heads_case(name, seed, b, L, h, p, g, chunk, full, with_seq_idx=False, cu_seqlens=None):
        """out and final_states of the reference's heads-style entry point for state size 1 and A = -1; with
        cu_seqlens (batch 1: packed sequences, seq_idx derived from it) also the state at the end of every sequence
        (return_varlen_states, kernels/ema_combined.py:56-62, kernels/ema_chunk_state.py:578)."""
        import kernels.ema_combined as ref_combined
        import kernels.ema_chunk_state as m1, kernels.ema_state_passing as m2, kernels.ema_bmm as m3, kernels.ema_chunk_scan as m4
        for mod in (m1, m2, m3, m4):
            for attr in dir(mod):
                k = getattr(mod, attr)
                if isinstance(getattr(k, "configs", None), list) and k.configs:
                    k.configs = k.configs[:1]
        rs = np.random.RandomState(seed)
        f32 = lambda a: np.ascontiguousarray(a, dtype=np.float32)
        rec = dict(x=f32(rs.standard_normal((b, L, h, p))), A=-np.ones(h, np.float32),
                   B=f32(rs.random_sample((b, L, g, 1))))
        if full:
            rec.update(dt=f32(0.3 * rs.standard_normal((b, L, h)) - 1.0), C=f32(0.5 + rs.random_sample((b, L, g, 1))),
                       D=f32(rs.standard_normal((h, p))), z=f32(rs.standard_normal((b, L, h, p))),
                       dt_bias=f32(0.1 * rs.standard_normal(h)), initial_states=f32(rs.standard_normal((b, h, p, 1))))
            kw = dict(dt_softplus=True, dt_limit=(0.001, 2.0))
        else:
            rec.update(dt=f32(0.01 + 0.2 * rs.random_sample((b, L, h))), C=np.ones((b, L, g, 1), np.float32))
            kw = {}
        if with_seq_idx:
            sid = np.zeros((b, L), np.int32)
            sid[0, L // 3:] = 1
            sid[0, chunk:] += 1          # a restart exactly on a chunk boundary
            sid[1, L - 7:] = 5
            rec["seq_idx"] = sid
        if cu_seqlens is not None:
            assert b == 1 and cu_seqlens[0] == 0 and cu_seqlens[-1] == L
            sid = np.zeros((1, L), np.int32)
            for i in range(len(cu_seqlens) - 1):
                sid[0, cu_seqlens[i]:cu_seqlens[i + 1]] = i
            rec["seq_idx"] = sid
            rec["cu_seqlens"] = np.asarray(cu_seqlens, np.int32)
        t = {k: torch.tensor(v) for k, v in rec.items()}
        with torch.no_grad():
            res = ref_combined.ema_chunk_scan_combined(
                t["x"], t["dt"], t["A"], t["B"], t["C"], chunk, D=t.get("D"), z=t.get("z"), dt_bias=t.get("dt_bias"),
                initial_states=t.get("initial_states"), seq_idx=t.get("seq_idx"), cu_seqlens=t.get("cu_seqlens"),
                return_final_states=True, return_varlen_states=cu_seqlens is not None, **kw)
        out, fin = res[0], res[1]
        if cu_seqlens is not None:
            rec["varlen_states"] = res[2].numpy()
        rec.update(out=out.numpy(), final_states=fin.numpy(), meta=np.array([seed, b, L, h, p, g, chunk, int(full)]),
                   meta_A_is_minus_one=np.array([1]))
        np.savez(os.path.join(args.out, name + ".npz"), **rec)
        print(name, "done", float(np.abs(rec["out"]).max()))

    if args.only == "heads_varlen":
        # (added after the other fixtures were recorded: --only leaves those files untouched)
        heads_case("heads_varlen", 24, 1, 120, 2, 16, 1, 32, full=False, cu_seqlens=[0, 37, 64, 101, 120])
        heads_case("heads_varlen_full", 25, 1, 100, 4, 16, 2, 32, full=True, cu_seqlens=[0, 5, 70, 100])
        return
    heads_case("heads_plain", 21, 2, 96, 2, 16, 1, 32, full=False)
    heads_case("heads_full", 22, 2, 100, 4, 16, 2, 32, full=True)
    heads_case("heads_seqidx", 23, 2, 90, 2, 16, 1, 32, full=False, with_seq_idx=True)
    heads_case("heads_varlen", 24, 1, 120, 2, 16, 1, 32, full=False, cu_seqlens=[0, 37, 64, 101, 120])
    heads_case("heads_varlen_full", 25, 1, 100, 4, 16, 2, 32, full=True, cu_seqlens=[0, 5, 70, 100])
    north_star_case("northstar_c1", 1235, 2, 256, 2, 64, 2.0, 6.0, per_head=False)
    north_star_case("northstar_perhead", 1237, 2, 192, 3, 32, 2.0, 6.0, per_head=True)
    north_star_case("northstar_ragged", 1241, 1, 77, 2, 24, 3.0, 8.0, per_head=False)
    stage_case("stages_ragged", 7, 3, 200, 24, 64, 0.1)
    stage_case("stages_even", 11, 2, 128, 32, 32, 1.0)


if __name__ == "__main__":
    main()
