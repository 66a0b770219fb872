"""Timing of the serialization gather and PointLiteConv kernels against their torch formulation
(models/dest_module.py:378-423) with CUDA events on the current stream:

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
    print(json.dumps(out))


if __name__ == "__main__":
    main()
