"""Timing of the serialization gather, PointLiteConv and dt / B / C generation kernels against their torch
formulation (models/dest_module.py:378-423, 541-559) with CUDA events on the current stream:

    python -m dest3d_b200.pointops_bench [--batch 64] [--points 16384] [--channels 290] [--reps 10] [--no-torch]

Inputs are larger than L2 at the default sizes.  Prints one JSON object; bandwidths are algorithmic bytes (each input
read once, each output written once) over the duration of the whole autograd call."""
import argparse
import json

import torch
import torch.nn.functional as F

from . import PointLiteConv, reorder_points


def _ms(fn, reps):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / reps


def glue(args):
    """dt / B / C (both directions) from dist (16 x 4096 points x 256 states x 16 features): forward, and backward to dist,
    the two projection weights and the per-token terms."""
    from .adaptive_params import adaptive_dt_bc
    b, L, K, M, H = min(args.batch, 16), 4096, 256, 16, 8
    gen = torch.Generator(device="cuda").manual_seed(1)
    res = {"batch": b, "points": L, "states": K, "features": M, "heads": H}
    for dt_, name in ((torch.bfloat16, "bf16"), (torch.float32, "f32")):
        rn = lambda *s: torch.randn(*s, device="cuda", generator=gen).to(dt_)
        dist = rn(b, L, K, M).requires_grad_(True)
        w_dt, w_bc = (rn(H, M).float() * 0.3).requires_grad_(True), (rn(2, M).float() * 0.3).requires_grad_(True)
        tok = [rn(b, L, H).requires_grad_(True)] + [rn(b, L, 1).requires_grad_(True) for _ in range(4)]
        bias = (rn(H).float() - 2.0).requires_grad_(True)
        mask = (torch.rand(b, L, K, device="cuda", generator=gen) > 0.3).float()
        leaves = [dist, w_dt, w_bc, bias] + tok

        def mine():
            return adaptive_dt_bc(dist, w_dt, w_bc, tok[0], bias, tok[1], tok[2], tok[3], tok[4], mask)

        def ref():
            bc = F.linear(dist, w_bc.to(dt_))
            bb, cb = bc[..., :1].transpose(-1, -2), bc[..., 1:].transpose(-1, -2)
            d = F.softplus(F.linear(dist, w_dt.to(dt_)).transpose(-1, -2) + tok[0].unsqueeze(-1) + bias.to(dt_).reshape(1, 1, -1, 1))
            return (d * mask.unsqueeze(2).to(dt_), bb + tok[1].unsqueeze(-1), cb + tok[2].unsqueeze(-1), bb + tok[3].unsqueeze(-1),
                    cb + tok[4].unsqueeze(-1))
        douts = [torch.randn_like(o) for o in mine()]
        es = dist.element_size()
        n = b * L * K
        fwd = _ms(mine, args.reps)
        bwd = _ms(lambda: torch.autograd.grad(mine(), leaves, douts), args.reps) - fwd
        r = {"fwd_ms": fwd, "fwd_gbs": n * (M + H + 4) * es / fwd / 1e6,                 # dist in; dt and four B / C rows out
             "bwd_ms": bwd, "bwd_gbs": n * (2 * M + H + 4) * es / bwd / 1e6}             # dist, ddt, dbc in; ddist out
        if not args.no_torch:
            tf = _ms(ref, args.reps)
            r["torch_fwd_ms"] = tf
            r["torch_bwd_ms"] = _ms(lambda: torch.autograd.grad(ref(), leaves, douts), args.reps) - tf
        res[name] = r
    return res


def norm(args):
    """z-gated RMSNorm (layernorm_gated.py:35-95) over 2^18 rows x 288 features, forward and backward, kernel launches
    only (preallocated leaves): the detector's key_norm at a size larger than L2."""
    from . import rmsnorm_fn
    rows, H = 1 << 18, 288
    gen = torch.Generator(device="cuda").manual_seed(2)
    res = {"rows": rows, "hidden": H}
    for dt_, name in ((torch.bfloat16, "bf16"), (torch.float32, "f32")):
        x = torch.randn(rows, H, device="cuda", generator=gen).to(dt_).requires_grad_(True)
        z = torch.randn(rows, H, device="cuda", generator=gen).to(dt_).requires_grad_(True)
        w = (1 + 0.02 * torch.randn(H, device="cuda", generator=gen)).requires_grad_(True)
        dy = torch.randn(rows, H, device="cuda", generator=gen).to(dt_)
        es = x.element_size()
        fwd = _ms(lambda: rmsnorm_fn(x, w, None, z, eps=1e-5, norm_before_gate=False), args.reps)
        bwd = _ms(lambda: torch.autograd.grad(rmsnorm_fn(x, w, None, z, eps=1e-5, norm_before_gate=False), (x, z, w), dy), args.reps) - fwd
        res[name] = {"fwd_ms": fwd, "fwd_gbs": 3 * rows * H * es / fwd / 1e6, "bwd_ms": bwd, "bwd_gbs": 5 * rows * H * es / bwd / 1e6}
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--points", type=int, default=16384)
    ap.add_argument("--channels", type=int, default=290)
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--no-torch", action="store_true", help="skip the torch formulation")
    args = ap.parse_args()
    B, N, C = args.batch, args.points, args.channels
    out = {"batch": B, "points": N, "channels": C}
    gen = torch.Generator(device="cuda").manual_seed(0)
    for dt, name in ((torch.bfloat16, "bf16"), (torch.float32, "f32")):
        x = torch.randn(B, N, C, device="cuda", generator=gen).to(dt).requires_grad_(True)
        dy = torch.randn(B, N, C, device="cuda", generator=gen).to(dt)
        mod = PointLiteConv(C, C).cuda()
        params = (x, mod.dwconv.weight, mod.dwconv.bias)
        es = x.element_size()
        fwd = _ms(lambda: mod(None, x), args.reps)
        bwd = _ms(lambda: torch.autograd.grad(mod(None, x), params, dy), args.reps) - fwd
        r = {"conv_fwd_ms": fwd, "conv_fwd_gbs": 2 * x.numel() * es / fwd / 1e6,
             "conv_bwd_ms": bwd, "conv_bwd_gbs": 3 * x.numel() * es / bwd / 1e6}
        order = torch.stack([torch.randperm(N, device="cuda") for _ in range(B)])
        pts = x.detach()
        g = _ms(lambda: reorder_points(pts, order), args.reps)
        r.update(gather_ms=g, gather_gbs=2 * pts.numel() * es / g / 1e6)
        if not args.no_torch:
            conv = torch.nn.Conv1d(C, C, 7, padding=3, groups=C).cuda().to(dt)

            def ref():
                return F.silu(conv(x.transpose(1, 2))).transpose(1, 2)
            tf = _ms(ref, args.reps)
            r["torch_conv_fwd_ms"] = tf
            r["torch_conv_bwd_ms"] = _ms(lambda: torch.autograd.grad(ref(), (x, conv.weight, conv.bias), dy), args.reps) - tf
            r["torch_gather_ms"] = _ms(lambda: pts.gather(1, order.unsqueeze(-1).expand(-1, -1, C)), args.reps)
        out[name] = r
    out["glue"] = glue(args)
    out["norm"] = norm(args)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
