"""Shared helpers of the parity tests: run the oracle and the CUDA path on the same seeded inputs.

Tolerances (from the benchmark definition): float32 rtol 1e-4 / atol 1e-5; bfloat16 inputs with
float32 accumulation rtol 1e-2 / atol 1e-2.  `atol` is applied relative to the largest magnitude
of the reference tensor (never below 1), because gradients such as dA are sums over batch x
seqlen whose absolute scale grows with the problem size:
    |got - ref| <= atol * max(1, max|ref|) + rtol * |ref|
"""
import torch

from oracle import issm_oracle as O

TOL = {torch.float32: (1e-4, 1e-5), torch.bfloat16: (1e-2, 1e-2)}
GRADS = ("x", "dt", "A", "B", "C", "D", "z", "dt_bias", "initial_states")


def close(got, ref, dtype, name, report=None, loosen=1.0):
    rtol, atol = TOL[dtype]
    rtol, atol = rtol * loosen, atol * loosen
    got = got.detach().double().cpu()
    ref = ref.detach().double().cpu()
    assert got.shape == ref.shape, f"{name}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    scale = max(1.0, ref.abs().max().item())
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
                    reverse=opts.get("reverse", False), compute_dtype=compute_dtype)
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
