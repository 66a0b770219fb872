"""Guard bands around every output and workspace of the kernels either side of the scan (row gather, PointLiteConv,
dt / B / C generation): the buffers are carved out of larger ones with a byte pattern on both sides and a NaN-filled
payload; after the call the margins are untouched and every output element is finite and right.  Shapes: ragged
segment tails, a single point, odd channel / state counts (scalar paths), widths that leave lanes idle."""
import pytest
import torch
import torch.nn.functional as F

from tests.test_canary_gpu import GuardedAllocator

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,N,C", [(1, 1, 2), (2, 67, 290), (1, 129, 33), (3, 16, 514), (1, 1030, 6)])
def test_conv_guard_bands(monkeypatch, dtype, B, N, C):
    from dest3d_b200 import pointops
    alloc = GuardedAllocator()
    monkeypatch.setattr(pointops, "_empty", alloc)
    g = torch.Generator().manual_seed(N + C)
    x = torch.randn(B, N, C, generator=g).to(dtype).cuda().requires_grad_()
    w = torch.randn(C, 1, 7, generator=g).cuda().requires_grad_()
    b = torch.randn(C, generator=g).cuda().requires_grad_()
    dy = torch.randn(B, N, C, generator=g).to(dtype).cuda()
    y = pointops.DwConv7SiluFn.apply(x, w, b)
    gx, gw, gb = torch.autograd.grad(y, (x, w, b), dy)
    alloc.check()
    x64, w64, b64 = (t.detach().double().cpu().requires_grad_() for t in (x, w, b))
    ref = F.silu(F.conv1d(x64.transpose(1, 2), w64, b64, padding=3, groups=C)).transpose(1, 2)
    rx, rw, rb = torch.autograd.grad(ref, (x64, w64, b64), dy.double().cpu())
    tol = dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=1e-4, atol=1e-5)
    for got, want in ((y, ref), (gx, rx)):
        assert torch.isfinite(got).all()
        torch.testing.assert_close(got.double().cpu(), want.detach(), **tol)
    for got, want in ((gw, rw), (gb, rb)):
        assert torch.isfinite(got).all()
        lim = (3e-2 if dtype == torch.bfloat16 else 1e-5) * (want.abs().max().item() + 1e-6)
        assert (got.double().cpu() - want).abs().max().item() <= lim


@pytest.mark.parametrize("dtype,B,N,M_,C", [(torch.bfloat16, 2, 100, 37, 290), (torch.float32, 1, 5, 5, 3), (torch.bfloat16, 1, 64, 64, 1),
                                            (torch.int64, 2, 33, 7, 6), (torch.bfloat16, 3, 40, 40, 288)])
def test_gather_guard_bands(monkeypatch, dtype, B, N, M_, C):
    from dest3d_b200 import pointops
    alloc = GuardedAllocator()
    g = torch.Generator().manual_seed(N + C)
    pts = (torch.randn(B, N, C, generator=g) * 50).to(dtype).cuda()
    idx = torch.randint(0, N, (B, M_), generator=g).cuda()
    if dtype == torch.int64:                                  # the NaN fill of the helper is for floating types
        raw = torch.full((4096 + B * M_ * C * 8 + 4096,), 0x5A, dtype=torch.uint8, device="cuda")
        monkeypatch.setattr(pointops, "_empty", lambda shape, dt, dev: raw[4096:4096 + B * M_ * C * 8].view(torch.int64).view(tuple(shape)))
        out = pointops.reorder_points(pts, idx, check=True)
        torch.cuda.synchronize()
        assert bool((raw[:4096] == 0x5A).all()) and bool((raw[4096 + B * M_ * C * 8:] == 0x5A).all())
    else:
        monkeypatch.setattr(pointops, "_empty", alloc)
        out = pointops.reorder_points(pts, idx, check=True)
        alloc.check()
    assert torch.equal(out, pts.gather(1, idx.unsqueeze(-1).expand(-1, -1, C)))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("b,L,K,M,H,G,back", [(1, 1, 256, 16, 8, 1, True), (2, 3, 131, 8, 2, 2, True), (1, 7, 600, 4, 4, 1, False),
                                              (1, 1300, 64, 16, 8, 1, True)])
def test_parameter_generation_guard_bands(monkeypatch, dtype, b, L, K, M, H, G, back):
    """More points than backward blocks (1300 > 1184), more states than one shared-memory tile (600 > 256), an odd
    state count (131: scalar stores, element-wise staging)."""
    from dest3d_b200 import adaptive_params as ap
    alloc = GuardedAllocator()
    monkeypatch.setattr(ap, "_empty", alloc)
    g = torch.Generator().manual_seed(L + K)
    rn = lambda *s: torch.randn(*s, generator=g)
    host = dict(dist=rn(b, L, K, M).to(dtype), w_dt=rn(H, M) * 0.3, w_bc=rn(2 * G, M) * 0.3, dt_tok=rn(b, L, H).to(dtype), dt_bias=rn(H) - 2.0,
                b_bias=rn(b, L, G).to(dtype), c_bias=rn(b, L, G).to(dtype))
    if back:
        host.update(b_back=rn(b, L, G).to(dtype), c_back=rn(b, L, G).to(dtype))
    mask = (torch.rand(b, L, K, generator=g) > 0.3).float()
    dev = {k: v.cuda().requires_grad_() for k, v in host.items()}
    outs = ap.adaptive_dt_bc(dev["dist"], dev["w_dt"], dev["w_bc"], dev["dt_tok"], dev["dt_bias"], dev["b_bias"], dev["c_bias"],
                             dev.get("b_back"), dev.get("c_back"), mask.cuda())
    douts = [rn(*o.shape) for o in outs]
    sum((o.float() * d.cuda()).sum() for o, d in zip(outs, douts)).backward()
    alloc.check()
    r = {k: v.double().requires_grad_() for k, v in host.items()}
    bc = F.linear(r["dist"], r["w_bc"])
    bb, cb = bc[..., :G].transpose(-1, -2), bc[..., G:].transpose(-1, -2)
    ref = [F.softplus(F.linear(r["dist"], r["w_dt"]).transpose(-1, -2) + r["dt_tok"].unsqueeze(-1) + r["dt_bias"].reshape(1, 1, -1, 1))
           * mask.unsqueeze(2), bb + r["b_bias"].unsqueeze(-1), cb + r["c_bias"].unsqueeze(-1)]
    if back:
        ref += [bb + r["b_back"].unsqueeze(-1), cb + r["c_back"].unsqueeze(-1)]
    sum((o * d.double()).sum() for o, d in zip(ref, douts)).backward()
    tol = dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=1e-4, atol=1e-5)
    for o, want in zip(outs, ref):
        assert torch.isfinite(o).all()
        torch.testing.assert_close(o.double().cpu(), want.detach(), **tol)
    for k in host:
        got, want = dev[k].grad.double().cpu(), r[k].grad
        assert torch.isfinite(got).all(), k
        if k == "dist":
            torch.testing.assert_close(got, want, **tol)
        else:
            assert (got - want).abs().max().item() <= (3e-2 if dtype == torch.bfloat16 else 1e-4) * (want.abs().max().item() + 1e-6), k
