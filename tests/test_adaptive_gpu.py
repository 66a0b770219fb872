"""dt / B / C generation from the distance features against the reference's own formulation
(models/dest_module.py:541-559: two Linear layers, transposes, per-token terms, softplus, mask), float64 on the CPU."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _reference(dist, w_dt, w_bc, dt_tok, dt_bias, b_bias, c_bias, b_back, c_back, mask, G):
    bc = F.linear(dist, w_bc)
    b_base, c_base = torch.split(bc, [G, G], dim=-1)
    out = [None, b_base.transpose(-1, -2) + b_bias.unsqueeze(-1), c_base.transpose(-1, -2) + c_bias.unsqueeze(-1)]
    if b_back is not None:
        out += [b_base.transpose(-1, -2) + b_back.unsqueeze(-1), c_base.transpose(-1, -2) + c_back.unsqueeze(-1)]
    dt = F.softplus(F.linear(dist, w_dt).transpose(-1, -2) + dt_tok.unsqueeze(-1) + dt_bias.reshape(1, 1, -1, 1))
    if mask is not None:
        if mask.dtype == torch.bool:
            dt = dt.masked_fill(mask.unsqueeze(2), 0.0)
        else:
            dt = dt * mask.unsqueeze(2).to(dt.dtype)
    out[0] = dt
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("b,L,K,M,H,G,back,mask", [
    (2, 37, 256, 16, 8, 1, True, "float"), (1, 5, 64, 4, 4, 1, False, None), (2, 9, 130, 8, 2, 2, True, "bool"),
    (1, 300, 256, 16, 8, 1, True, None)])
def test_adaptive_dt_bc_matches_reference_formulation(dtype, b, L, K, M, H, G, back, mask):
    from dest3d_b200.adaptive_params import adaptive_dt_bc
    g = torch.Generator().manual_seed(b * 100 + L + K + M)
    rn = lambda *s: torch.randn(*s, generator=g)
    host = dict(dist=rn(b, L, K, M).to(dtype), w_dt=rn(H, M) * 0.3, w_bc=rn(2 * G, M) * 0.3, dt_tok=rn(b, L, H).to(dtype),
                dt_bias=rn(H) - 2.0, b_bias=rn(b, L, G).to(dtype), c_bias=rn(b, L, G).to(dtype))
    if back:
        host.update(b_back=rn(b, L, G).to(dtype), c_back=rn(b, L, G).to(dtype))
    m = None
    if mask == "float":
        m = (torch.rand(b, L, K, generator=g) > 0.3).float()
    elif mask == "bool":
        m = torch.rand(b, L, K, generator=g) > 0.7
    dev = {k: v.cuda().requires_grad_() for k, v in host.items()}
    got = adaptive_dt_bc(dev["dist"], dev["w_dt"], dev["w_bc"], dev["dt_tok"], dev["dt_bias"], dev["b_bias"], dev["c_bias"],
                         dev.get("b_back"), dev.get("c_back"), None if m is None else m.cuda())
    ref_in = {k: v.double().requires_grad_() for k, v in host.items()}
    ref = _reference(ref_in["dist"], ref_in["w_dt"], ref_in["w_bc"], ref_in["dt_tok"], ref_in["dt_bias"], ref_in["b_bias"],
                     ref_in["c_bias"], ref_in.get("b_back"), ref_in.get("c_back"), m, G)
    assert len(got) == len(ref) == (5 if back else 3)
    assert got[0].shape == (b, L, H, K) and got[1].shape == (b, L, G, K)
    tol = dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=1e-4, atol=1e-5)
    douts = [rn(*r.shape) for r in ref]
    for o, r in zip(got, ref):
        torch.testing.assert_close(o.double().cpu(), r.detach(), **tol)
    sum((o.float() * d.cuda()).sum() for o, d in zip(got, douts)).backward()
    sum((r * d.double()).sum() for r, d in zip(ref, douts)).backward()
    for k in host:
        gg, gr = dev[k].grad.double().cpu(), ref_in[k].grad
        if k == "dist":
            torch.testing.assert_close(gg, gr, **tol)
        else:                                               # sums over many (point, state) pairs: relative to the largest entry
            lim = (3e-2 if dtype == torch.bfloat16 else 1e-4) * (gr.abs().max().item() + 1e-6)
            assert (gg - gr).abs().max().item() <= lim, k


def test_outputs_feed_the_scan_without_copies():
    """dt is contiguous (b, L, H, K) and B / C are row-strided views the tensor-core path reads through TMA tiles."""
    from dest3d_b200 import ISSM_chunk_scan_combined
    from dest3d_b200.adaptive_params import adaptive_dt_bc
    g = torch.Generator().manual_seed(1)
    b, L, K, M, H, P = 1, 200, 256, 16, 2, 36
    rn = lambda *s: torch.randn(*s, generator=g).cuda().bfloat16()
    dt, B, C = adaptive_dt_bc(rn(b, L, K, M), rn(H, M).float() * 0.2, rn(2, M).float() * 0.1, rn(b, L, H), torch.full((H,), -3.0).cuda(),
                              rn(b, L, 1), rn(b, L, 1))
    assert dt.is_contiguous() and B.stride(1) == 2 * K
    A = -torch.rand(H, K, generator=g).cuda() - 0.5
    x = rn(b, L, H, P)
    y = ISSM_chunk_scan_combined(x, dt, A, B, C, 64, path="tensor")
    y2 = ISSM_chunk_scan_combined(x, dt, A, B.contiguous(), C.contiguous(), 64, path="tensor")
    assert torch.equal(y, y2)


@pytest.mark.parametrize("b,L,K,M,H,G,back", [(2, 37, 256, 16, 8, 1, True), (1, 9, 130, 8, 2, 2, False), (1, 300, 256, 4, 4, 1, True)])
def test_float_features_with_bfloat16_outputs(b, L, K, M, H, G, back):
    """What autocast hands the block: dist stays float32, dt / B / C come out in bfloat16, ddist goes back in float32."""
    from dest3d_b200.adaptive_params import adaptive_dt_bc
    g = torch.Generator().manual_seed(L + K)
    rn = lambda *s: torch.randn(*s, generator=g)
    host = dict(dist=rn(b, L, K, M), w_dt=rn(H, M) * 0.3, w_bc=rn(2 * G, M) * 0.3, dt_tok=rn(b, L, H).bfloat16(), dt_bias=rn(H) - 2.0,
                b_bias=rn(b, L, G).bfloat16(), c_bias=rn(b, L, G).bfloat16())
    if back:
        host.update(b_back=rn(b, L, G).bfloat16(), c_back=rn(b, L, G).bfloat16())
    m = (torch.rand(b, L, K, generator=g) > 0.3).float()
    dev = {k: v.cuda().requires_grad_() for k, v in host.items()}
    got = adaptive_dt_bc(dev["dist"], dev["w_dt"], dev["w_bc"], dev["dt_tok"], dev["dt_bias"], dev["b_bias"], dev["c_bias"],
                         dev.get("b_back"), dev.get("c_back"), m.cuda(), out_dtype=torch.bfloat16)
    assert all(o.dtype == torch.bfloat16 for o in got)
    r = {k: v.double().requires_grad_() for k, v in host.items()}
    ref = _reference(r["dist"], r["w_dt"], r["w_bc"], r["dt_tok"], r["dt_bias"], r["b_bias"], r["c_bias"], r.get("b_back"), r.get("c_back"), m, G)
    douts = [rn(*o.shape) for o in ref]
    for o, want in zip(got, ref):
        torch.testing.assert_close(o.double().cpu(), want.detach(), rtol=2e-2, atol=2e-2)
    sum((o.float() * d.cuda()).sum() for o, d in zip(got, douts)).backward()
    sum((o * d.double()).sum() for o, d in zip(ref, douts)).backward()
    assert dev["dist"].grad.dtype == torch.float32
    # the incoming gradients are rounded to bfloat16 on their way into the kernel; everything else is float32
    torch.testing.assert_close(dev["dist"].grad.double().cpu(), r["dist"].grad, rtol=2e-2, atol=2e-2)
    for k in host:
        if k != "dist":
            want = r[k].grad
            assert (dev[k].grad.double().cpu() - want).abs().max().item() <= 3e-2 * (want.abs().max().item() + 1e-6), k
    with pytest.raises(TypeError):
        adaptive_dt_bc(dev["dist"].detach().bfloat16(), dev["w_dt"], dev["w_bc"], dev["dt_tok"], dev["dt_bias"], dev["b_bias"], dev["c_bias"],
                       out_dtype=torch.float32)
