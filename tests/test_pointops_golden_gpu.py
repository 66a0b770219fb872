"""The CUDA kernels either side of the scan against outputs of the REFERENCE's own code (tests/golden/pointops_golden.npz,
written by tests/golden/make_golden_pointops.py from PointLiteConv, Serialization.reorder_points and the dt / B / C lines
of MultiHeadISSMScan.forward), and against the oracle restatement on larger seeded inputs."""
import os

import numpy as np
import pytest
import torch

from oracle import pointops_oracle as P

pytestmark = pytest.mark.gpu
F32 = dict(rtol=1e-4, atol=1e-5)


def _golden():
    path = os.path.join(os.path.dirname(__file__), "golden", "pointops_golden.npz")
    return {k: torch.from_numpy(v) for k, v in np.load(path).items()}


def test_point_lite_conv_against_the_reference_fixture():
    from dest3d_b200 import PointLiteConv
    g = _golden()
    mod = PointLiteConv(10, 10)
    mod.load_state_dict({"dwconv.weight": g["conv_w"].float(), "dwconv.bias": g["conv_b"].float()})
    mod = mod.cuda()
    x = g["conv_x"].float().cuda().requires_grad_()
    y = mod(None, x)
    torch.testing.assert_close(y.double().cpu(), g["conv_y"], **F32)
    gx, gw, gb = torch.autograd.grad(y, (x, mod.dwconv.weight, mod.dwconv.bias), g["conv_dy"].float().cuda())
    for got, want in ((gx, g["conv_dx"]), (gw, g["conv_dw"]), (gb, g["conv_db"])):
        torch.testing.assert_close(got.double().cpu(), want, **F32)


def test_reorder_points_against_the_reference_fixture():
    from dest3d_b200 import reorder_points
    g = _golden()
    out = reorder_points(g["gather_points"].cuda(), g["gather_index"].cuda(), g["gather_inverse"].cuda(), check=True)
    assert torch.equal(out.cpu(), g["gather_out"])                         # float64 rows, copied byte for byte
    assert torch.equal(reorder_points(out, g["gather_inverse"].cuda()).cpu(), g["gather_points"])


def test_parameter_generation_against_the_reference_fixture():
    from dest3d_b200.adaptive_params import adaptive_dt_bc
    g = _golden()
    c = lambda k: g[k].float().cuda()
    outs = adaptive_dt_bc(c("glue_dist"), c("glue_w_dt"), c("glue_w_bc"), c("glue_dt_tok"), c("glue_dt_bias"), c("glue_b_bias"),
                          c("glue_c_bias"), c("glue_b_back"), c("glue_c_back"), c("glue_mask"))
    for got, name in zip(outs, ("glue_dt", "glue_B", "glue_C", "glue_B_back", "glue_C_back")):
        torch.testing.assert_close(got.double().cpu(), g[name], **F32)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_kernels_against_the_oracle_restatement(dtype):
    """Seeded inputs of the detector's widths through the oracle (float64, explicit index arithmetic) and the kernels."""
    from dest3d_b200 import PointLiteConv, reorder_points
    from dest3d_b200.adaptive_params import adaptive_dt_bc
    gen = torch.Generator().manual_seed(21)
    rn = lambda *s: torch.randn(*s, generator=gen)
    tol = F32 if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    x, w, b = rn(2, 300, 290).to(dtype), rn(290, 1, 7) * 0.3, rn(290) * 0.3
    mod = PointLiteConv(290, 290)
    mod.load_state_dict({"dwconv.weight": w, "dwconv.bias": b})
    y = mod.cuda()(None, x.cuda())
    torch.testing.assert_close(y.double().cpu(), P.point_lite_conv(x.double(), w.double(), b.double()), **tol)
    idx = torch.stack([torch.randperm(300, generator=gen) for _ in range(2)])
    assert torch.equal(reorder_points(x.cuda(), idx.cuda()).cpu(), P.reorder_points(x, idx))
    dist, w_dt, w_bc = rn(2, 40, 256, 16).to(dtype), rn(8, 16) * 0.3, rn(2, 16) * 0.3
    tok, bias, bb, cb = rn(2, 40, 8).to(dtype), rn(8) - 2, rn(2, 40, 1).to(dtype), rn(2, 40, 1).to(dtype)
    mask = torch.rand(2, 40, 256, generator=gen) > 0.8                     # bool: True zeroes dt
    got = adaptive_dt_bc(dist.cuda(), w_dt.cuda(), w_bc.cuda(), tok.cuda(), bias.cuda(), bb.cuda(), cb.cuda(), mask=mask.cuda())
    want = P.adaptive_dt_bc(dist.double(), w_dt.double(), w_bc.double(), tok.double(), bias.double(), bb.double(), cb.double(), mask=mask)
    for a, r in zip(got, want):
        torch.testing.assert_close(a.double().cpu(), r, **tol)
