"""GPU parity of the gated RMS / Layer norm against the oracle and the reference's golden vectors."""
import os

import numpy as np
import pytest
import torch

from oracle import issm_oracle as O
from tests import parity

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("is_rms", [True, False], ids=["rms", "ln"])
@pytest.mark.parametrize("nbg", [False, True], ids=["gate_first", "norm_first"])
@pytest.mark.parametrize("gs", [None, 36])
@pytest.mark.parametrize("use_z", [True, False], ids=["z", "noz"])
def test_norm_parity(dtype, is_rms, nbg, gs, use_z):
    from dest3d_b200 import layernorm_fn
    g = torch.Generator().manual_seed(3)
    x = torch.randn(7, 33, 288, generator=g).to(dtype)
    z = torch.randn(7, 33, 288, generator=g).to(dtype) if use_z else None
    w = 1 + 0.02 * torch.randn(288, generator=g)
    bias = None if is_rms else 0.1 * torch.randn(288, generator=g)
    dy = torch.randn(7, 33, 288, generator=g).to(dtype)
    ref_l = [t.double().requires_grad_() if t is not None else None for t in (x, w, bias, z)]
    # oracle in float64 on the (possibly bf16-rounded) inputs
    xr, wr, br, zr = ref_l
    xf = xr if not (use_z and not nbg) else xr * torch.nn.functional.silu(zr)
    grp = 288 if gs is None else gs
    xg = xf.reshape(7, 33, 288 // grp, grp)
    if is_rms:
        xh = xg * torch.rsqrt(xg.square().mean(-1, keepdim=True) + 1e-5)
    else:
        xc = xg - xg.mean(-1, keepdim=True)
        xh = xc * torch.rsqrt(xc.square().mean(-1, keepdim=True) + 1e-5)
    yr = xh.reshape(7, 33, 288) * wr + (br if br is not None else 0)
    if use_z and nbg:
        yr = yr * torch.nn.functional.silu(zr)
    (yr * dy.double()).sum().backward()
    # float32 oracle restatement must agree with this float64 formula too
    yo = O.gated_norm_ref(x, w, bias, z, eps=1e-5, group_size=gs, norm_before_gate=nbg, is_rms_norm=is_rms)
    parity.close(yo, yr, dtype, "oracle_y")
    leaves = [t.cuda().requires_grad_() if t is not None else None for t in (x, w, bias, z)]
    xc_, wc, bc, zc = leaves
    y = layernorm_fn(xc_, wc, bc, zc, eps=1e-5, group_size=gs, norm_before_gate=nbg, is_rms_norm=is_rms)
    (y.float() * dy.cuda().float()).sum().backward()
    parity.close(y, yr, dtype, "y")
    parity.close(xc_.grad, xr.grad, dtype, "dx")
    parity.close(wc.grad, wr.grad, dtype, "dw")
    if bias is not None:
        parity.close(bc.grad, br.grad, dtype, "db")
    if use_z:
        parity.close(zc.grad, zr.grad, dtype, "dz")


def test_rmsnorm_reference_golden():
    from dest3d_b200 import rmsnorm_fn
    g = np.load(os.path.join(GOLD, "rmsnorm_gated.npz"))
    x, z, w = (torch.from_numpy(g[k]).cuda() for k in ("x", "z", "w"))
    for nbg in (False, True):
        for gs in (None, 36):
            for use_z in (True, False):
                key = f"nbg{int(nbg)}_gs{gs or 0}_z{int(use_z)}"
                xr, zr, wr = x.clone().requires_grad_(), z.clone().requires_grad_(), w.clone().requires_grad_()
                y = rmsnorm_fn(xr, wr, None, zr if use_z else None, eps=1e-5, group_size=gs, norm_before_gate=nbg)
                (y * torch.cos(torch.arange(y.numel(), dtype=torch.float32, device="cuda").reshape(y.shape))).sum().backward()
                parity.close(y, torch.from_numpy(g["y_" + key]), torch.float32, "y_" + key)
                parity.close(xr.grad, torch.from_numpy(g["dx_" + key]), torch.float32, "dx_" + key)
                parity.close(wr.grad, torch.from_numpy(g["dw_" + key]), torch.float32, "dw_" + key)
                if use_z:
                    parity.close(zr.grad, torch.from_numpy(g["dz_" + key]), torch.float32, "dz_" + key)


def test_module_interface_and_determinism():
    from dest3d_b200 import RMSNorm
    m = RMSNorm(288, eps=1e-5, norm_before_gate=False, device="cuda")
    assert m.bias is None and list(m.state_dict().keys()) == ["weight"]
    x = torch.randn(4, 1000, 288, device="cuda", requires_grad=True)
    z = torch.randn(4, 1000, 288, device="cuda")
    y1 = m(x, z)
    y1.sum().backward()
    g1, w1 = x.grad.clone(), m.weight.grad.clone()
    x.grad = None
    m.weight.grad = None
    y2 = m(x, z)
    y2.sum().backward()
    assert torch.equal(y1, y2) and torch.equal(g1, x.grad) and torch.equal(w1, m.weight.grad)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("nbg", [False, True], ids=["gate_first", "norm_first"])
def test_gate_as_a_column_slice_of_the_projection(dtype, nbg):
    """The detector's gate: z = zxbcdt[..., :288] of a (b, L, 586) projection output (models/dest_module.py:528-529),
    rows 1172 bytes apart in bfloat16, i.e. starting 4 bytes off a 16-byte boundary; also a slice that starts inside
    the row.  Same results as with a contiguous copy, bit for bit (the vector kernels read such a gate as 4-byte words)."""
    from dest3d_b200 import _lib, rmsnorm_fn
    g = torch.Generator().manual_seed(8)
    x = torch.randn(5, 40, 288, generator=g).to(dtype).cuda().requires_grad_()
    wide = torch.randn(5, 40, 586, generator=g).to(dtype).cuda()
    w = (1 + 0.02 * torch.randn(288, generator=g)).cuda().requires_grad_()
    dy = torch.randn(5, 40, 288, generator=g).to(dtype).cuda()
    for lo in (0, 2):
        zv = wide[..., lo:lo + 288].detach().requires_grad_()          # a leaf that is itself a strided view
        zc = wide[..., lo:lo + 288].contiguous().requires_grad_()
        n0 = _lib.launch_count()
        y1 = rmsnorm_fn(x, w, None, zv, eps=1e-5, norm_before_gate=nbg)
        g1 = torch.autograd.grad(y1, (x, w, zv), dy)
        used = _lib.launch_count() - n0
        y2 = rmsnorm_fn(x, w, None, zc, eps=1e-5, norm_before_gate=nbg)
        g2 = torch.autograd.grad(y2, (x, w, zc), dy)
        assert torch.equal(y1, y2)
        for a, b in zip(g1, g2):
            assert torch.equal(a, b)
        assert used == 3                                        # forward, backward, one fixed-order reduction
