"""Generates tests/golden/pointops_golden.npz from the REFERENCE's own code for the steps either side of the scan.

    python tests/golden/make_golden_pointops.py REF_DIR      (a checkout of the reference)

* `PointLiteConv` (models/dest_module.py:400-423): forward and the gradients of input, weight and bias, float64.
* `Serialization.reorder_points` / `reversed_reorder_points` (:378-397), called on a stand-in object that only carries
  the index lists (the class's constructor needs the detector's Hilbert template file, which is not part of the path).
* The dt / B / C generation (:541-559): `MultiHeadISSMScan.forward` is run unmodified in float64 with the scan call
  replaced by a recorder, so the stored dt, B, C, B_back, C_back are exactly what the reference hands its scan; the
  per-token terms are read off the reference's own intermediate results with forward hooks.
`timm` (one unused import of the reference file) is stubbed.  Nothing from this repository takes part in the numbers."""
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden_pointops.py REF_DIR   (a checkout of the reference)")
    timm, tm, tl = types.ModuleType("timm"), types.ModuleType("timm.models"), types.ModuleType("timm.models.layers")
    tl.DropPath = torch.nn.Identity
    timm.models, tm.layers = tm, tl
    sys.modules.update({"timm": timm, "timm.models": tm, "timm.models.layers": tl})
    sys.path.insert(0, sys.argv[1])
    import models.dest_module as dm

    torch.manual_seed(7)
    out = {}
    # ---- PointLiteConv ----
    conv = dm.PointLiteConv(10, 10).double()
    x = torch.randn(2, 23, 10, dtype=torch.float64, requires_grad=True)
    dy = torch.randn(2, 23, 10, dtype=torch.float64)
    y = conv(torch.zeros(2, 23, 3), x)
    gx, gw, gb = torch.autograd.grad(y, (x, conv.dwconv.weight, conv.dwconv.bias), dy)
    out.update(conv_x=x.detach(), conv_w=conv.dwconv.weight.detach(), conv_b=conv.dwconv.bias.detach(), conv_dy=dy, conv_y=y.detach(),
               conv_dx=gx, conv_dw=gw, conv_db=gb)
    # ---- Serialization gather ----
    pts = torch.randn(2, 19, 5, dtype=torch.float64)
    order = torch.stack([torch.randperm(19) for _ in range(2)])
    inverse = torch.empty_like(order).scatter_(1, order, torch.arange(19).expand(2, 19))
    holder = types.SimpleNamespace(index_list=[order], reversed_index_list=[inverse])
    fwd = dm.Serialization.reorder_points(holder, pts)
    back = dm.Serialization.reversed_reorder_points(holder, fwd)
    assert torch.equal(back, pts)
    out.update(gather_points=pts, gather_index=order, gather_inverse=inverse, gather_out=fwd)
    # ---- dt / B / C as the reference's block hands them to its scan ----
    b, L, K, d_model, M, H = 2, 12, 16, 8, 16, 4
    mod = dm.MultiHeadISSMScan(d_model=d_model, d_state=K, d_dist=M, chunk_size=K, nheads=H, expand=2, use_biscan=True).double()
    seen, inter = [], {}

    def recorder(xx, dt, A, B, C, chunk_size=None, D=None, z=None, initial_states=None, **kw):
        seen.append((dt.detach().clone(), B.detach().clone(), C.detach().clone()))
        return torch.zeros_like(xx), torch.zeros(xx.shape[0], xx.shape[2], xx.shape[3], A.shape[1], dtype=xx.dtype)

    dm.ISSM_chunk_scan_combined = recorder

    class Skip(torch.nn.Module):                                           # the gated norm (a Triton kernel) is not part of these lines
        def forward(self, key, z=None):
            return key

    mod.key_norm = Skip()
    hooks = [mod.key_proj.register_forward_hook(lambda m, i, o: inter.__setitem__("zxbcdt", o.detach())),
             mod.key_conv.register_forward_hook(lambda m, i, o: inter.__setitem__("xbc", o.detach())),
             mod.key_conv_back.register_forward_hook(lambda m, i, o: inter.__setitem__("xbc_back", o.detach()))]
    in_key, in_query = torch.randn(b, L, d_model, dtype=torch.float64), torch.randn(b, K, d_model, dtype=torch.float64)
    dist, xyz = torch.randn(b, L, K, M, dtype=torch.float64), torch.randn(b, L, 3, dtype=torch.float64)
    mask = (torch.rand(b, L, K) > 0.25).float()
    with torch.no_grad():
        mod(in_key, in_query, dist, xyz, mask)
    for h in hooks:
        h.remove()
    d_inner = mod.d_inner
    (dt, B, C), (dt_flipped, B_back_flipped, C_back_flipped) = seen       # the second call gets flipped tensors (:567-571)
    assert torch.equal(torch.flip(dt_flipped, dims=[1]), dt)
    out.update(glue_dist=dist, glue_mask=mask, glue_w_dt=mod.dt_proj.weight.detach(), glue_w_bc=mod.bc_proj.weight.detach(),
               glue_dt_bias=mod.dt_bias.detach(), glue_dt_tok=inter["zxbcdt"][..., -H:],
               glue_b_bias=inter["xbc"][..., d_inner:d_inner + 1], glue_c_bias=inter["xbc"][..., d_inner + 1:d_inner + 2],
               glue_b_back=inter["xbc_back"][..., d_inner:d_inner + 1], glue_c_back=inter["xbc_back"][..., d_inner + 1:d_inner + 2],
               glue_dt=dt, glue_B=B, glue_C=C, glue_B_back=torch.flip(B_back_flipped, dims=[1]), glue_C_back=torch.flip(C_back_flipped, dims=[1]))
    np.savez_compressed(os.path.join(HERE, "pointops_golden.npz"), **{k: (v.numpy() if torch.is_tensor(v) else v) for k, v in out.items()})
    print("wrote pointops_golden.npz with", sorted(out))


if __name__ == "__main__":
    main()
