"""Generates the golden fixtures in this directory from the REFERENCE's own pure-PyTorch code.

    python tests/golden/make_golden.py REF_DIR      (a checkout of the reference)

`ISSM_minimal_discrete` (test_issm.py:18-67) and `rms_norm_ref`
(issm_triton/layernorm_gated.py:8-29) are imported unmodified; nothing from this repository
takes part in producing the numbers.  Small cases store inputs and every output / gradient in
full; the reference's own test shape (test_issm.py:74-77, seed 42) stores outputs in full and
the large gradients subsampled, with inputs regenerated from the seed by `case_inputs` below
(an input checksum is stored to detect generator drift).
"""
import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))

# (name, b, L, H, P, N, Q, seed, dtype)
CASES = [
    ("tiny_f64", 1, 64, 2, 4, 16, 16, 1, torch.float64),
    ("ragged_heads_f64", 2, 96, 3, 5, 8, 32, 2, torch.float64),
    ("reftest_f32", 1, 512, 8, 32, 256, 256, 42, torch.float32),
]
SUB = 4  # subsampling stride for the big gradients of the reference test shape


def case_inputs(b, L, H, P, N, seed, dtype):
    """Same recipe as test_issm.py:79-86 (dt = softplus(randn - 4), A = -exp(rand) of shape
    (H, N)), drawn from a seeded CPU generator so tests can regenerate them."""
    g = torch.Generator().manual_seed(seed)
    mk = lambda *s: torch.randn(*s, generator=g, dtype=dtype)
    x, Bm, Cm = mk(b, L, H, P), mk(b, L, 1, N), mk(b, L, 1, N)
    dt = F.softplus(mk(b, L, H, N) - 4)
    A = -torch.exp(torch.rand(H, N, generator=g, dtype=dtype))
    s0 = mk(b, H, P, N)
    w = mk(b, L, H, P)
    wf = mk(b, H, P, N)
    return dict(x=x, B=Bm, C=Cm, dt=dt, A=A, init=s0, w=w, wf=wf)


def main():
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py REF_DIR   (a checkout of the reference)")
    ref_dir = sys.argv[1]
    sys.path.insert(0, ref_dir)
    from test_issm import ISSM_minimal_discrete
    from issm_triton.layernorm_gated import rms_norm_ref

    for name, b, L, H, P, N, Q, seed, dtype in CASES:
        inp = case_inputs(b, L, H, P, N, seed, dtype)
        leaves = {k: inp[k].clone().requires_grad_() for k in ("x", "dt", "A", "B", "C", "init")}
        y, fin = ISSM_minimal_discrete(leaves["x"], leaves["dt"], leaves["A"] * leaves["dt"],
                                       leaves["B"].expand(b, L, H, N), leaves["C"].expand(b, L, H, N), Q,
                                       initial_states=leaves["init"])
        ((y * inp["w"]).sum() + (fin * inp["wf"]).sum()).backward()
        big = name == "reftest_f32"
        out = dict(shape=np.array([b, L, H, P, N, Q, seed]), y=y.detach().numpy(), final=fin.detach().numpy())
        out["input_checksum"] = np.array([float(sum(inp[k].double().sum() for k in ("x", "B", "C", "dt", "A", "init")))])
        for k in leaves:
            gk = leaves[k].grad.numpy()
            if big and gk.size > 70000:
                gk = gk.reshape(-1)[::SUB]
            out["d" + k] = gk
        if not big:
            for k in inp:
                out["in_" + k] = inp[k].numpy()
        out = {k: (v.astype(np.float32) if v.dtype == np.float64 and k != "input_checksum" else v) for k, v in out.items()}
        np.savez_compressed(os.path.join(HERE, f"issm_{name}.npz"), **out)
        print(name, {k: v.shape for k, v in out.items()})

    # gated RMS norm fixtures (DEST's configuration first: norm_before_gate=False, no groups)
    g = torch.Generator().manual_seed(11)
    x = torch.randn(6, 9, 288, generator=g)
    z = torch.randn(6, 9, 288, generator=g)
    w = 1.0 + 0.02 * torch.randn(288, generator=g)
    out = dict(x=x.numpy(), z=z.numpy(), w=w.numpy())
    for nbg in (False, True):
        for gs in (None, 36):
            for use_z in (True, False):
                xr, zr, wr = x.clone().requires_grad_(), z.clone().requires_grad_(), w.clone().requires_grad_()
                y = rms_norm_ref(xr, wr, None, z=zr if use_z else None, eps=1e-5, group_size=gs, norm_before_gate=nbg)
                (y * torch.cos(torch.arange(y.numel(), dtype=torch.float32).reshape(y.shape))).sum().backward()
                key = f"nbg{int(nbg)}_gs{gs or 0}_z{int(use_z)}"
                out["y_" + key] = y.detach().numpy()
                out["dx_" + key] = xr.grad.numpy()
                out["dw_" + key] = wr.grad.numpy()
                if use_z:
                    out["dz_" + key] = zr.grad.numpy()
    np.savez_compressed(os.path.join(HERE, "rmsnorm_gated.npz"), **out)
    print("rmsnorm", len(out))


if __name__ == "__main__":
    main()
