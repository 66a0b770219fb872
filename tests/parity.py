"""Shared helpers of the parity tests: run the oracle and the CUDA path on the same seeded inputs.

Tolerances (from the benchmark definition): float32 rtol 1e-4 / atol 1e-5; bfloat16 inputs with
float32 accumulation rtol 1e-2 / atol 1e-2.

Per-point tensors (out, final states, dx, dz, dinitial_states: values of order one) are held to the
literal bound
    |got - ref| <= atol + rtol * |ref|
Reductions over many points (ddt chains a reverse cumulative sum through the block; dA, dB, dC, dD,
ddt_bias sum over heads, batch and sequence) have an absolute scale that grows with the problem size,
so for them `atol` is applied relative to the largest magnitude of the reference tensor (never below 1):
    |got - ref| <= atol * max(1, max|ref|) + rtol * |ref|
Every comparison appends (name, max error, scale used, worst error / bound) to the report, so a test
can print which tensors needed a scale above one.
"""
import torch

from oracle import issm_oracle as O

TOL = {torch.float32: (1e-4, 1e-5), torch.bfloat16: (1e-2, 1e-2)}
GRADS = ("x", "dt", "A", "B", "C", "D", "z", "dt_bias", "initial_states")
# tensors held to the literal tolerance (no scaling by the reference's magnitude)
LITERAL = ("out", "final", "dx", "dz", "dinitial_states")


def close(got, ref, dtype, name, report=None, loosen=1.0, literal=None):
    rtol, atol = TOL[dtype]
    rtol, atol = rtol * loosen, atol * loosen
    got = got.detach().double().cpu()
    ref = ref.detach().double().cpu()
    assert got.shape == ref.shape, f"{name}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    if literal is None:
        literal = name in LITERAL
    scale = 1.0 if literal else max(1.0, ref.abs().max().item() if ref.numel() else 0.0)
    err = (got - ref).abs()
    bound = atol * scale + rtol * ref.abs()
    worst = (err / bound).max().item() if err.numel() else 0.0
    if report is not None:
        report.append((name, err.max().item() if err.numel() else 0.0, scale, worst))
    assert torch.isfinite(got).all(), f"{name}: non-finite values"
    assert worst <= 1.0, f"{name}: max err {err.max().item():.3e} (scale {scale:.3e}) exceeds tolerance x{worst:.2f}"


def oracle_run(inp, Q, opts, compute_dtype=torch.float64, scan=None):
    """Oracle forward + autograd backward on CPU.  Returns dict(out, final, d<name>...)."""
    scan = scan or O.issm_scan_chunked
    leaves = {}
    for k in GRADS:
        v = inp.get(k)
        if v is not None and opts.get("use_" + k, True):
            leaves[k] = v.detach().clone().to(compute_dtype).requires_grad_()
    use = lambda k: leaves.get(k)
    out, fin = scan(leaves["x"], leaves["dt"], leaves["A"], leaves["B"], leaves["C"], Q, D=use("D"), z=use("z"),
                    dt_bias=use("dt_bias"), initial_states=use("initial_states"),
                    dt_softplus=opts.get("dt_softplus", False), dt_limit=opts.get("dt_limit", (0.0, float("inf"))),
                    reverse=opts.get("reverse", False), compute_dtype=compute_dtype, **opts.get("scan_kw", {}))
    loss = (out * inp["dout"].to(out.dtype)).sum()
    if opts.get("dfinal", True):
        loss = loss + (fin * inp["dfinal"].to(fin.dtype)).sum()
    loss.backward()
    res = {"out": out.detach(), "final": fin.detach()}
    for k, v in leaves.items():
        res["d" + k] = v.grad
    return res


def cuda_run(inp, Q, opts, path="auto", device="cuda"):
    """The product path through the public Python interface (which calls the C ABI)."""
    from dest3d_b200 import ISSM_chunk_scan_combined
    leaves = {}
    for k in GRADS:
        v = inp.get(k)
        if v is not None and opts.get("use_" + k, True):
            t = v.detach().clone().to(device)
            if opts.get("noncontig") and k in ("x", "z"):
                # a (b, L, H*P) buffer viewed as (b, L, H, P) inside a wider row, as rearrange() of a
                # split projection produces (models/dest_module.py:531,601)
                b, L, H, P = t.shape
                wide = torch.zeros(b, L, H * P + 8, dtype=t.dtype, device=device)
                wide[..., 4:4 + H * P] = t.reshape(b, L, H * P)
                t = wide[..., 4:4 + H * P].unflatten(-1, (H, P))
            if opts.get("noncontig_bc") and k in ("B", "C"):
                # B and C as the two halves of one projection output, as torch.split() leaves them: row stride 2 N
                bb, L, G, N = t.shape
                wide = torch.zeros(bb, L, G, 2 * N, dtype=t.dtype, device=device)
                half = slice(0, N) if k == "B" else slice(N, 2 * N)
                wide[..., half] = t
                t = wide[..., half]
            leaves[k] = t.requires_grad_()
    use = lambda k: leaves.get(k)
    want_final = opts.get("return_final", True)
    res = ISSM_chunk_scan_combined(leaves["x"], leaves["dt"], leaves["A"], leaves["B"], leaves["C"], Q, D=use("D"),
                                   z=use("z"), dt_bias=use("dt_bias"), initial_states=use("initial_states"),
                                   dt_softplus=opts.get("dt_softplus", False),
                                   dt_limit=opts.get("dt_limit", (0.0, float("inf"))),
                                   return_final_states=want_final, reverse=opts.get("reverse", False), path=path)
    out, fin = res if want_final else (res, None)
    loss = (out.float() * inp["dout"].to(device).float()).sum()
    if want_final and opts.get("dfinal", True):
        loss = loss + (fin * inp["dfinal"].to(device)).sum()
    loss.backward()
    r = {"out": out.detach(), "final": None if fin is None else fin.detach()}
    for k, v in leaves.items():
        r["d" + k] = v.grad
    return r


def compare(got, ref, dtype, want_final=True, loosen=1.0):
    report = []
    close(got["out"], ref["out"], dtype, "out", report, loosen)
    if want_final:
        close(got["final"], ref["final"], dtype, "final", report, loosen)
    for k in ref:
        if k.startswith("d"):
            assert got.get(k) is not None, f"{k}: gradient missing"
            close(got[k], ref[k], dtype, k, report, loosen)
    return report


def oracle_run_sliced(inp, Q, opts, compute_dtype=torch.float64, scan=None):
    """`oracle_run` evaluated one (sample, head) stream at a time, so that the oracle's O(states x Q^2)
    intermediates of a long sequence stay within a few GB: the loss is a sum over streams, per-stream
    gradients are written to their slice, parameter gradients (dA, dD, ddt_bias) and the gradients of the
    head-shared B and C are accumulated.  Single group only (B, C shared by every head)."""
    b, L, H, P = inp["x"].shape
    assert inp["B"].shape[2] == 1
    res = None
    per_stream = {"x": (0, 2), "dt": (0, 2), "z": (0, 2), "initial_states": (0, 1)}   # (batch dim, head dim)
    per_head = {"A": 0, "D": 0, "dt_bias": 0}
    for bi in range(b):
        for h in range(H):
            sl = {}
            for k, v in inp.items():
                if not torch.is_tensor(v):
                    sl[k] = v
                elif k in per_stream or k == "dout":
                    bd, hd = per_stream.get(k, (0, 2))
                    sl[k] = v.narrow(bd, bi, 1).narrow(hd, h, 1)
                elif k == "dfinal":
                    sl[k] = v[bi:bi + 1, h:h + 1]
                elif k in per_head:
                    sl[k] = v[h:h + 1]
                else:                                       # B, C
                    sl[k] = v[bi:bi + 1]
            r = oracle_run(sl, Q, opts, compute_dtype, scan)
            if res is None:
                res = {"out": torch.zeros(b, L, H, P, dtype=r["out"].dtype), "final": torch.zeros(b, H, P, inp["B"].shape[-1], dtype=r["final"].dtype)}
                for k, v in r.items():
                    if k.startswith("d"):
                        full = inp[k[1:]]
                        res[k] = torch.zeros(full.shape, dtype=v.dtype)
            res["out"][bi:bi + 1, :, h:h + 1] = r["out"]
            res["final"][bi:bi + 1, h:h + 1] = r["final"]
            for k, v in r.items():
                if not k.startswith("d"):
                    continue
                name = k[1:]
                if name in per_stream:
                    bd, hd = per_stream[name]
                    res[k].narrow(bd, bi, 1).narrow(hd, h, 1).copy_(v)
                elif name in per_head:
                    res[k][h:h + 1] += v
                else:
                    res[k][bi:bi + 1] += v
    return res


def format_report(report):
    """One line per compared tensor: worst error / bound, and the scale when it is not one."""
    return ", ".join(f"{n} x{w:.2f}" + (f" (scale {s:.3g})" if s != 1.0 else "") for n, _, s, w in report)
