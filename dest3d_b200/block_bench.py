"""Forward + backward of one whole ISSM block (`MultiHeadISSMScan`, models/dest_module.py:426-612) at the detector's
size, CUDA events:  python -m dest3d_b200.block_bench [--batch 8] [--points 1024] [--reference <checkout or copy>]

Times this library's block (`dest3d_b200.issm_block`) and, when a copy of the reference is given (default
baseline/_ref beside the package, if present), the reference's own module class with only its two imports served by
this library (scan and gated norm on the CUDA kernels, everything else in torch) on the same inputs and weights."""
import argparse
import importlib
import json
import os
import sys
import types

import torch


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


def _reference_class(ref_dir):
    here = os.path.dirname(os.path.abspath(__file__))
    if not os.path.isfile(os.path.join(ref_dir, "models", "dest_module.py")):
        return None
    timm, tm, tl = types.ModuleType("timm"), types.ModuleType("timm.models"), types.ModuleType("timm.models.layers")
    tl.DropPath = torch.nn.Identity
    timm.models, tm.layers = tm, tl
    sys.modules.setdefault("timm", timm)
    sys.modules.setdefault("timm.models", tm)
    sys.modules.setdefault("timm.models.layers", tl)
    sys.path[:0] = [os.path.join(here, "shim"), ref_dir]
    return importlib.import_module("models.dest_module").MultiHeadISSMScan


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--points", type=int, default=1024)
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--graph", action="store_true", help="also time the step replayed from a CUDA graph")
    ap.add_argument("--reference", default=os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref"))
    args = ap.parse_args()
    from .issm_block import MultiHeadISSMScan
    b, L, K, d_model, M, H = args.batch, args.points, 256, 144, 16, 8
    kw = dict(d_model=d_model, d_state=K, d_dist=M, chunk_size=K, nheads=H, expand=2, use_biscan=True)
    torch.manual_seed(0)
    mine = MultiHeadISSMScan(**kw).cuda()
    g = torch.Generator(device="cuda").manual_seed(0)
    rn = lambda *s: torch.randn(*s, device="cuda", generator=g)
    in_key, in_query, dist, xyz = rn(b, L, d_model).requires_grad_(), (rn(b, K, d_model) / 4).requires_grad_(), rn(b, L, K, M).requires_grad_(), rn(b, L, 3)
    mask = (torch.rand(b, L, K, device="cuda", generator=g) > 0.1).float()
    gk, gq = rn(b, L, d_model), rn(b, K, d_model)

    def step(mod):
        def run():
            with torch.autocast("cuda", dtype=torch.bfloat16):
                ok, oq = mod(in_key, in_query, dist, xyz, mask)
            ((ok.float() * gk).sum() + (oq.float() * gq).sum()).backward()
            mod.zero_grad(set_to_none=True)
            in_key.grad = in_query.grad = dist.grad = None     # assigned, not accumulated, in the next step
        return run

    out = {"batch": b, "points": L, "states": K, "d_model": d_model, "dtype": "bf16 autocast",
           "native_block_ms": _ms(step(mine), args.reps)}
    if args.graph:
        # the same step captured once into a CUDA graph and replayed (the step is launch-bound at the detector's size)
        run = step(mine)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                run()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            run()
        out["native_block_graph_replay_ms"] = _ms(graph.replay, args.reps)
    ref_cls = _reference_class(args.reference)
    if ref_cls is not None:
        ref = ref_cls(**kw)
        ref.load_state_dict(mine.state_dict())
        out["reference_module_with_library_scan_and_norm_ms"] = _ms(step(ref.cuda()), args.reps)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
