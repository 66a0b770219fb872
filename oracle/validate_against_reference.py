"""Pins oracle/issm_oracle.py against the reference's own pure-PyTorch code.

Run in a container that has the reference checkout:  python oracle/validate_against_reference.py REF_DIR
It imports `ISSM_minimal_discrete` (test_issm.py:18-67) and `rms_norm_ref`
(issm_triton/layernorm_gated.py:8-29) UNMODIFIED and compares outputs and autograd gradients
with the restatement on seeded inputs.  Exit code 0 = every check passed.
"""
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
from oracle import issm_oracle as O  # noqa: E402


def load_reference(ref_dir):
    sys.path.insert(0, ref_dir)
    from test_issm import ISSM_minimal_discrete  # noqa
    from issm_triton.layernorm_gated import rms_norm_ref  # noqa
    return ISSM_minimal_discrete, rms_norm_ref


def check(name, a, b, rtol, atol):
    ok = torch.allclose(a, b, rtol=rtol, atol=atol)
    err = (a - b).abs().max().item()
    print(f"{'ok ' if ok else 'BAD'} {name}: max abs diff {err:.3e}")
    return ok


def main():
    if len(sys.argv) != 2:
        raise SystemExit("usage: python oracle/validate_against_reference.py REF_DIR   (a checkout of the reference, "
                         "or the copy made by oracle/install_reference.py under baseline/_ref)")
    ref_dir = sys.argv[1]
    ref_scan, ref_norm = load_reference(ref_dir)
    ok = True
    for dtype, rtol, atol in ((torch.float64, 1e-10, 1e-12), (torch.float32, 1e-4, 1e-5)):
        for (b, L, H, P, N, Q, seed) in ((1, 64, 2, 4, 16, 16, 1), (2, 96, 3, 5, 8, 32, 2), (1, 512, 8, 32, 256, 256, 42)):
            if dtype == torch.float64 and N == 256:
                continue
            g = torch.Generator().manual_seed(seed)
            mk = lambda *s: torch.randn(*s, generator=g, dtype=dtype)
            x, Bm, Cm = mk(b, L, H, P), mk(b, L, 1, N), mk(b, L, 1, N)
            dt = torch.nn.functional.softplus(mk(b, L, H, N) - 4)
            A = -torch.exp(torch.rand(H, N, generator=g, dtype=dtype))
            s0 = mk(b, H, P, N)
            leaves_ref = [t.clone().requires_grad_() for t in (x, dt, A, Bm, Cm, s0)]
            xr, dtr, Ar, Br, Cr, sr = leaves_ref
            y_ref, f_ref = ref_scan(xr, dtr, Ar * dtr, Br.expand(b, L, H, N), Cr.expand(b, L, H, N), Q, initial_states=sr)
            leaves = [t.clone().requires_grad_() for t in (x, dt, A, Bm, Cm, s0)]
            xo, dto, Ao, Bo, Co, so = leaves
            y, f = O.issm_scan_chunked(xo, dto, Ao, Bo, Co, Q, initial_states=so, compute_dtype=dtype)
            y2, f2 = O.issm_scan_sequential(x, dt, A, Bm, Cm, initial_states=s0, compute_dtype=torch.float64)
            tag = f"{str(dtype)[6:]} b{b} L{L} H{H} P{P} N{N} Q{Q}"
            ok &= check(f"out   {tag}", y, y_ref, rtol, atol)
            ok &= check(f"final {tag}", f.to(dtype), f_ref, rtol, atol)
            ok &= check(f"out   {tag} (recurrence vs reference)", y2.to(dtype), y_ref.detach(), rtol * 10, atol * 10)
            w = torch.randn(y.shape, generator=g, dtype=dtype)
            wf = torch.randn(f.shape, generator=g, dtype=dtype)
            ((y_ref * w).sum() + (f_ref * wf).sum()).backward()
            ((y * w).sum() + (f.to(dtype) * wf).sum()).backward()
            for nm, a_, b_ in zip(("dx", "ddt", "dA", "dB", "dC", "dinit"), leaves, leaves_ref):
                scale = b_.grad.abs().max().item()
                ok &= check(f"{nm:5s} {tag}", a_.grad / scale, b_.grad / scale, rtol * 10, atol * 10)
    # gated RMS norm
    g = torch.Generator().manual_seed(7)
    x = torch.randn(5, 7, 48, generator=g)
    z = torch.randn(5, 7, 48, generator=g)
    w = torch.randn(48, generator=g)
    bias = torch.randn(48, generator=g)
    for nbg in (True, False):
        for gs in (None, 16):
            for zz in (None, z):
                for bb in (None, bias):
                    r = ref_norm(x, w, bb, z=zz, eps=1e-5, group_size=gs, norm_before_gate=nbg)
                    o = O.gated_norm_ref(x, w, bb, z=zz, eps=1e-5, group_size=gs, norm_before_gate=nbg, is_rms_norm=True)
                    ok &= check(f"rmsnorm nbg={nbg} gs={gs} z={zz is not None} bias={bb is not None}", o, r, 1e-6, 1e-6)
    print("ALL OK" if ok else "MISMATCH")
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
