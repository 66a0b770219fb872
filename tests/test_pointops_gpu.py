"""Serialization gather and PointLiteConv on the GPU against the reference's own formulation in torch
(models/dest_module.py:378-423): points.gather(dim=1, tiled index) and SiLU(Conv1d(k=7, pad=3, groups=C)) on the
transposed tensor, evaluated on the CPU in float64."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _ref_conv(x, w, b):
    y = F.conv1d(x.transpose(1, 2), w, b, padding=3, groups=x.shape[2])
    return F.silu(y).transpose(1, 2)


def _tol(dtype):
    return dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,N,C", [(2, 1024, 290), (1, 5, 8), (3, 130, 33), (1, 64, 2), (2, 67, 514)])
def test_point_lite_conv_matches_torch(dtype, B, N, C):
    from dest3d_b200 import PointLiteConv
    torch.manual_seed(B * 1000 + N + C)
    mod = PointLiteConv(C, C).cuda()
    x = torch.randn(B, N, C, device="cuda").to(dtype).requires_grad_(True)
    dy = torch.randn(B, N, C, device="cuda").to(dtype)
    y = mod(None, x)
    assert y.shape == (B, N, C) and y.dtype == dtype
    y.backward(dy)

    w64 = mod.dwconv.weight.detach().double().cpu().requires_grad_(True)
    b64 = mod.dwconv.bias.detach().double().cpu().requires_grad_(True)
    x64 = x.detach().double().cpu().requires_grad_(True)
    y64 = _ref_conv(x64, w64, b64)
    y64.backward(dy.double().cpu())
    t = _tol(dtype)
    torch.testing.assert_close(y.double().cpu(), y64.detach(), **t)
    torch.testing.assert_close(x.grad.double().cpu(), x64.grad, **t)
    # reductions over B * N rows: tolerance relative to the largest entry
    for got, ref in ((mod.dwconv.weight.grad, w64.grad), (mod.dwconv.bias.grad, b64.grad)):
        scale = ref.abs().max().item() + 1e-6
        lim = (2e-2 if dtype == torch.bfloat16 else 1e-5) * scale
        assert (got.double().cpu() - ref).abs().max().item() <= lim


def test_point_lite_conv_strided_input_and_determinism():
    from dest3d_b200.pointops import DwConv7SiluFn
    torch.manual_seed(3)
    big = torch.randn(2, 300, 640, device="cuda")
    x = big[:, :, 100:390]                                   # row stride 640, channel stride 1
    w = torch.randn(290, 1, 7, device="cuda", requires_grad=True)
    b = torch.randn(290, device="cuda", requires_grad=True)
    y = DwConv7SiluFn.apply(x, w, b)
    ref = _ref_conv(x.double().cpu(), w.detach().double().cpu(), b.detach().double().cpu())
    torch.testing.assert_close(y.double().cpu(), ref, rtol=1e-4, atol=1e-5)
    g1 = torch.autograd.grad(y.sum(), (w, b), retain_graph=True)
    g2 = torch.autograd.grad(y.sum(), (w, b))
    assert all(torch.equal(a, c) for a, c in zip(g1, g2))


def test_reference_state_dict_loads():
    from dest3d_b200 import PointLiteConv
    ref = torch.nn.Conv1d(16, 16, kernel_size=7, padding=3, groups=16)
    mod = PointLiteConv(16, 16)
    mod.load_state_dict({"dwconv.weight": ref.weight.detach(), "dwconv.bias": ref.bias.detach()})
    mod = mod.cuda()
    x = torch.randn(2, 40, 16, device="cuda")
    want = F.silu(ref(x.cpu().transpose(1, 2))).transpose(1, 2)
    torch.testing.assert_close(mod(None, x).cpu(), want, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int64])
@pytest.mark.parametrize("B,N,C", [(2, 1024, 288), (1, 7, 3), (3, 100, 1), (2, 513, 6)])
def test_reorder_points_is_bit_exact(dtype, B, N, C):
    from dest3d_b200 import reorder_points
    g = torch.Generator().manual_seed(B + N + C)
    pts = (torch.randn(B, N, C, generator=g) * 100).to(dtype).cuda()
    order = torch.stack([torch.randperm(N, generator=g) for _ in range(B)]).cuda()
    inverse = torch.empty_like(order).scatter_(1, order, torch.arange(N, device="cuda").expand(B, N))
    got = reorder_points(pts, order, check=True)
    want = pts.gather(1, order.unsqueeze(-1).expand(-1, -1, C))
    assert torch.equal(got, want)
    # reorder followed by the reversed reorder is the identity (models/dest_module.py:388-397)
    assert torch.equal(reorder_points(got, inverse), pts)


def test_reorder_points_gradients_and_subset():
    from dest3d_b200 import reorder_points
    g = torch.Generator().manual_seed(5)
    B, N, C = 2, 257, 36
    pts = torch.randn(B, N, C, generator=g).cuda().requires_grad_(True)
    order = torch.stack([torch.randperm(N, generator=g) for _ in range(B)]).cuda()
    inverse = torch.empty_like(order).scatter_(1, order, torch.arange(N, device="cuda").expand(B, N))
    dy = torch.randn(B, N, C, generator=g).cuda()
    (gp,) = torch.autograd.grad(reorder_points(pts, order, inverse), pts, dy)
    (gr,) = torch.autograd.grad(pts.gather(1, order.unsqueeze(-1).expand(-1, -1, C)), pts, dy)
    assert torch.equal(gp, gr)
    # repeated indices, fewer rows than the source, no inverse: scatter-add adjoint
    idx = torch.randint(0, N, (B, 100), generator=g).cuda()
    (gp,) = torch.autograd.grad(reorder_points(pts, idx), pts, dy[:, :100])
    (gr,) = torch.autograd.grad(pts.gather(1, idx.unsqueeze(-1).expand(-1, -1, C)), pts, dy[:, :100])
    torch.testing.assert_close(gp, gr, rtol=1e-6, atol=1e-6)


def test_reorder_points_flags_an_index_out_of_range():
    from dest3d_b200 import reorder_points
    pts = torch.randn(1, 10, 4, device="cuda")
    idx = torch.tensor([[0, 3, 10]], device="cuda")
    with pytest.raises(IndexError):
        reorder_points(pts, idx, check=True)
    torch.cuda.synchronize()                                 # the context is intact
    assert torch.equal(reorder_points(pts, idx[:, :2], check=True), pts[:, [0, 3]])
