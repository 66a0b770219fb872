"""CPU oracle for the ISSM chunked scan and the gated norms.  TEST INFRASTRUCTURE ONLY.

This module is the checker the CUDA path is compared against.  It is never imported by the
product package; only the test-suite, the smoke entry and the CPU-baseline / reference legs of
the benchmark may call it.

Parity status: PINNED.  `oracle/validate_against_reference.py` compares every function here
with the reference's own pure-PyTorch code (`test_issm.py:18-67` ISSM_minimal_discrete and
`issm_triton/layernorm_gated.py:8-29` rms_norm_ref) imported unmodified, and the fixtures under
`tests/golden/` were produced by that reference code (see `tests/golden/make_golden.py`).

What is restated, and the reference lines each piece follows:

* chunked scan                      test_issm.py:18-67 (segsum :7-16)
* dt transform (bias, softplus with threshold 20, clamp, zero padding)
                                     issm_triton/issm_chunk_state.py:84-99, issm_triton/softplus.py:9-11
* D skip                             issm_triton/issm_chunk_scan.py:196-200
* z gate inside the scan             issm_triton/issm_chunk_scan.py:205-210
* output / final state dtypes        issm_triton/issm_combined.py:57-92
* gated RMS / Layer norm             issm_triton/layernorm_gated.py:8-29, 35-95
* bidirectional combine              models/dest_module.py:567-575

Two independent formulations are given (chunked, and the plain step-by-step recurrence); they
must agree, which guards the restatement itself.  Gradients come from torch autograd through
either formulation, exactly as the reference obtains its own reference gradients
(test_issm.py:100-104).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------------------
# dt transform
# --------------------------------------------------------------------------------------
def softplus_ref(v: torch.Tensor) -> torch.Tensor:
    """softplus with the reference's threshold: v if v > 20 else log(exp(v) + 1)
    (issm_triton/softplus.py:9-11)."""
    return torch.where(v <= 20.0, torch.log(torch.exp(torch.clamp(v, max=20.0)) + 1.0), v)


def dt_transform(dt, dt_bias=None, dt_softplus=False, dt_limit=(0.0, float("inf"))):
    """dt (b, L, H, N) -> transformed dt in the compute dtype
    (issm_triton/issm_chunk_state.py:84-98).  dt_bias is (H, N) or (H,)."""
    v = dt
    if dt_bias is not None:
        bias = dt_bias.to(v.dtype)
        if bias.dim() == 1:
            bias = bias[:, None]
        v = v + bias
    if dt_softplus:
        v = softplus_ref(v)
    lo, hi = dt_limit
    # the reference clamps unconditionally, so with the default (0, inf) a negative dt becomes 0;
    # torch.clamp passes the gradient on [lo, hi] inclusive, matching the strict outside-mask of
    # issm_chunk_state.py:212-216
    return torch.clamp(v, min=lo, max=hi)


def _expand_groups(t: torch.Tensor, nheads: int) -> torch.Tensor:
    """(b, L, G, N) -> (b, L, H, N); head h uses group h // (H / G)."""
    g = t.shape[2]
    if g == nheads:
        return t
    return t.repeat_interleave(nheads // g, dim=2)


def _prep(x, dt, A, B, C, D, z, dt_bias, initial_states, dt_softplus, dt_limit, compute_dtype):
    cd = compute_dtype
    H = x.shape[2]
    xs = x.to(cd)
    dtv = dt_transform(dt.to(cd), None if dt_bias is None else dt_bias.to(cd), dt_softplus, dt_limit)
    Av = A.to(cd)
    Bv = _expand_groups(B.to(cd), H)
    Cv = _expand_groups(C.to(cd), H)
    Dv = None if D is None else D.to(cd)
    zv = None if z is None else z.to(cd)
    s0 = None if initial_states is None else initial_states.to(cd)
    return xs, dtv, Av, Bv, Cv, Dv, zv, s0


def _epilogue(y, xs, Dv, zv):
    if Dv is not None:
        y = y + xs * (Dv[None, None, :, None] if Dv.dim() == 1 else Dv[None, None])
    if zv is not None:
        y = y * (zv * torch.sigmoid(zv))
    return y


# --------------------------------------------------------------------------------------
# formulation 1: the chunked algorithm of the reference oracle
# --------------------------------------------------------------------------------------
def _segsum(v: torch.Tensor) -> torch.Tensor:
    """out[..., i, j] = sum_{j < k <= i} v[..., k] for j <= i, -inf above the diagonal
    (test_issm.py:7-16)."""
    T = v.shape[-1]
    cs = torch.cumsum(v, dim=-1)
    d = cs[..., :, None] - cs[..., None, :]
    keep = torch.tril(torch.ones(T, T, dtype=torch.bool, device=v.device))
    return d.masked_fill(~keep, -float("inf"))


def _round_through(t: torch.Tensor, dtype) -> torch.Tensor:
    """Value rounded to `dtype`, gradient passed straight through (how a kernel that evaluates an
    analytic gradient formula on rounded operands behaves)."""
    return t + (t.detach().to(dtype).to(t.dtype) - t.detach())


def issm_scan_chunked(x, dt, A, B, C, chunk_size, D=None, z=None, dt_bias=None,
                      initial_states=None, dt_softplus=False, dt_limit=(0.0, float("inf")),
                      reverse=False, compute_dtype=torch.float32, operand_rounding=None):
    """Chunked ISSM scan.  Same argument meaning as ISSM_chunk_scan_combined
    (issm_triton/issm_combined.py:16-35) plus `reverse` (scan from the last point to the first;
    equal to flipping x, dt, B, C, z along L, scanning, and flipping the output back, which is
    what models/dest_module.py:567-573 does).

    Returns (out (b, L, H, P) in x.dtype, final_states (b, H, P, N) float32 [compute dtype if
    float64]).  Differentiable with torch autograd.

    `operand_rounding=torch.bfloat16` emulates what the reference's Triton kernels do to the intra-chunk
    term when B or C is bfloat16: the cumulative decay `a`, dt, B and C are all cast to the dot dtype before
    exp(a[l] - a[s]) * B * dt * C is formed (issm_triton/issm_cabt_bmm.py:40-43,124-136).  Only used by the
    tests that put this library's rounding error next to the reference's own.
    """
    if reverse:
        flip = lambda t: None if t is None else torch.flip(t, dims=[1])
        out, fin = issm_scan_chunked(flip(x), flip(dt), A, flip(B), flip(C), chunk_size, D, flip(z),
                                     dt_bias, initial_states, dt_softplus, dt_limit, False, compute_dtype,
                                     operand_rounding)
        return torch.flip(out, dims=[1]), fin
    b, L, H, P = x.shape
    N = B.shape[-1]
    Q = chunk_size
    xs, dtv, Av, Bv, Cv, Dv, zv, s0 = _prep(x, dt, A, B, C, D, z, dt_bias, initial_states,
                                            dt_softplus, dt_limit, compute_dtype)
    pad = (-L) % Q
    if pad:
        # tail padding: dt = 0 (decay 1, no input) and x = 0 (issm_chunk_state.py:99)
        padrows = lambda t: F.pad(t, (0, 0, 0, 0, 0, pad))
        xp, dtp, Bp, Cp = padrows(xs), padrows(dtv), padrows(Bv), padrows(Cv)
    else:
        xp, dtp, Bp, Cp = xs, dtv, Bv, Cv
    nc = (L + pad) // Q
    xc = xp.reshape(b, nc, Q, H, P)
    dtc = dtp.reshape(b, nc, Q, H, N)
    Bc = Bp.reshape(b, nc, Q, H, N)
    Cc = Cp.reshape(b, nc, Q, H, N)
    dA = dtc * Av[None, None, None]                       # (b, nc, Q, H, N)
    a = torch.cumsum(dA, dim=2)                           # in-chunk inclusive cumsum
    a_last = a[:, :, -1]                                  # (b, nc, H, N)

    # intra-chunk term, one head at a time to bound memory (the reference builds a
    # (b, H, N, nc, Q, Q) tensor in one go, test_issm.py:40)
    y_diag = []
    for h in range(H):
        if operand_rounding is None:
            seg = _segsum(dA[:, :, :, h].permute(0, 1, 3, 2))      # (b, nc, N, Q, Q)
            Lmat = torch.exp(seg)
            cabt = torch.einsum("bcln,bcsn,bcnls,bcsn->bcls", Cc[:, :, :, h], Bc[:, :, :, h], Lmat, dtc[:, :, :, h])
        else:
            rt = lambda t: _round_through(t, operand_rounding)
            ar = rt(a[:, :, :, h]).permute(0, 1, 3, 2)             # (b, nc, N, Q): the rounded cumulative decay
            keep = torch.tril(torch.ones(Q, Q, dtype=torch.bool))
            Lmat = rt(torch.exp((ar[..., :, None] - ar[..., None, :]).masked_fill(~keep, -float("inf"))))
            cabt = torch.einsum("bcln,bcsn,bcnls,bcsn->bcls", rt(Cc[:, :, :, h]), rt(Bc[:, :, :, h]), Lmat, rt(dtc[:, :, :, h]))
        y_diag.append(torch.einsum("bcls,bcsp->bclp", cabt, xc[:, :, :, h]))
    y = torch.stack(y_diag, dim=3)                        # (b, nc, Q, H, P)

    # per-chunk states and the inter-chunk recurrence
    decay_states = torch.exp(a_last[:, :, None] - a)      # (b, nc, Q, H, N)
    states = torch.einsum("bclhn,bclhn,bclhn,bclhp->bchpn", Bc, decay_states, dtc, xc)
    S = torch.zeros(b, H, P, N, dtype=xs.dtype) if s0 is None else s0
    entering = []
    for c in range(nc):
        entering.append(S)
        S = S * torch.exp(a_last[:, c])[:, :, None, :] + states[:, c]
    S_in = torch.stack(entering, dim=1)                   # (b, nc, H, P, N)
    y = y + torch.einsum("bclhn,bchpn,bclhn->bclhp", Cc, S_in, torch.exp(a))
    y = y.reshape(b, nc * Q, H, P)[:, :L]
    y = _epilogue(y, xs, Dv, zv)
    fin = S if compute_dtype == torch.float64 else S.float()
    return y.to(x.dtype if compute_dtype != torch.float64 else torch.float64), fin


# --------------------------------------------------------------------------------------
# formulation 2: the step-by-step recurrence the chunked algorithm implements
#   S_l = S_{l-1} * exp(dt_l * A) + x_l (outer) (B_l * dt_l);   y_l = S_l . C_l
# --------------------------------------------------------------------------------------
def issm_scan_sequential(x, dt, A, B, C, chunk_size=None, D=None, z=None, dt_bias=None,
                         initial_states=None, dt_softplus=False, dt_limit=(0.0, float("inf")),
                         reverse=False, compute_dtype=torch.float64):
    """Plain recurrence, independent of chunking; used to cross-check the chunked formulation and
    as the long-sequence oracle (memory O(b H P N)).  Differentiable."""
    b, L, H, P = x.shape
    N = B.shape[-1]
    xs, dtv, Av, Bv, Cv, Dv, zv, s0 = _prep(x, dt, A, B, C, D, z, dt_bias, initial_states,
                                            dt_softplus, dt_limit, compute_dtype)
    S = torch.zeros(b, H, P, N, dtype=xs.dtype) if s0 is None else s0
    ys = [None] * L
    order = range(L - 1, -1, -1) if reverse else range(L)
    for l in order:
        decay = torch.exp(dtv[:, l] * Av[None])                         # (b, H, N)
        S = S * decay[:, :, None, :] + xs[:, l][..., None] * (Bv[:, l] * dtv[:, l])[:, :, None, :]
        ys[l] = torch.einsum("bhpn,bhn->bhp", S, Cv[:, l])
    y = torch.stack(ys, dim=1)
    y = _epilogue(y, xs, Dv, zv)
    fin = S if compute_dtype == torch.float64 else S.float()
    return y.to(x.dtype if compute_dtype != torch.float64 else torch.float64), fin


# --------------------------------------------------------------------------------------
# bidirectional combine (models/dest_module.py:565-575)
# --------------------------------------------------------------------------------------
def issm_scan_bidirectional(x_f, x_b, dt, A, B_f, C_f, B_b, C_b, chunk_size, D=None, z=None,
                            dt_bias=None, initial_states=None, dt_softplus=False,
                            dt_limit=(0.0, float("inf")), out_scale=0.5,
                            scan=issm_scan_chunked, compute_dtype=torch.float32):
    """Forward scan of (x_f, B_f, C_f) plus reversed scan of (x_b, B_b, C_b) with the same dt,
    A, D and initial states; both results scaled by out_scale (0.5 = the reference's average)."""
    yf, sf = scan(x_f, dt, A, B_f, C_f, chunk_size, D, z, dt_bias, initial_states, dt_softplus,
                  dt_limit, False, compute_dtype)
    yb, sb = scan(x_b, dt, A, B_b, C_b, chunk_size, D, z, dt_bias, initial_states, dt_softplus,
                  dt_limit, True, compute_dtype)
    return ((yf.float() + yb.float()) * out_scale).to(x_f.dtype), (sf + sb) * out_scale


# --------------------------------------------------------------------------------------
# gated norms (issm_triton/layernorm_gated.py:8-29 for RMS; :35-95 for the LayerNorm variant)
# --------------------------------------------------------------------------------------
def gated_norm_ref(x, weight, bias=None, z=None, eps=1e-6, group_size=None,
                   norm_before_gate=True, is_rms_norm=True):
    """norm(x) * silu(z) if norm_before_gate else norm(x * silu(z)); statistics per group of
    `group_size` features (all features when None); computed in float32, returned in x.dtype."""
    dtype = x.dtype
    xf = x.float()
    w = weight.float()
    zf = None if z is None else z.float()
    if zf is not None and not norm_before_gate:
        xf = xf * F.silu(zf)
    Nf = xf.shape[-1]
    g = Nf if group_size is None else group_size
    xg = xf.reshape(*xf.shape[:-1], Nf // g, g)
    if is_rms_norm:
        rstd = torch.rsqrt(xg.square().mean(dim=-1, keepdim=True) + eps)
        xhat = xg * rstd
    else:
        mean = xg.mean(dim=-1, keepdim=True)
        xc = xg - mean
        rstd = torch.rsqrt(xc.square().mean(dim=-1, keepdim=True) + eps)
        xhat = xc * rstd
    out = xhat.reshape(xf.shape) * w
    if bias is not None:
        out = out + bias.float()
    if zf is not None and norm_before_gate:
        out = out * F.silu(zf)
    return out.to(dtype)


# --------------------------------------------------------------------------------------
# seeded synthetic inputs shared by tests, smoke and bench (value distributions of the
# benchmark configurations: x, z ~ N(0,1); B, C ~ N(0,1)/sqrt(N); dt_raw ~ N(0,1) with bias -4,
# softplus, clamp [1e-3, 1e-1]; A = -exp(U(log 1, log 16)) per head; D ~ N(0,1))
# --------------------------------------------------------------------------------------
def make_inputs(b, L, H, P, N, G=1, seed=0, dtype=torch.float32, with_z=True, with_init=True,
                D_has_hdim=False):
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g)
    x = rn(b, L, H, P)
    z = rn(b, L, H, P) if with_z else None
    Bm = rn(b, L, G, N) / math.sqrt(N)
    Cm = rn(b, L, G, N) / math.sqrt(N)
    dt = rn(b, L, H, N)
    A_head = -torch.exp(torch.rand(H, generator=g) * (math.log(16.0) - math.log(1.0)))
    A = A_head[:, None].repeat(1, N).contiguous()
    D = rn(H, P) if D_has_hdim else rn(H)
    dt_bias = torch.full((H, N), -4.0)
    init = rn(b, H, P, N) / 16.0 if with_init else None
    dout = rn(b, L, H, P)
    dfinal = rn(b, H, P, N) / 16.0
    cast = lambda t: None if t is None else t.to(dtype)
    return dict(x=cast(x), z=cast(z), B=cast(Bm), C=cast(Cm), dt=cast(dt), A=A, D=D, dt_bias=dt_bias,
                initial_states=cast(init), dout=cast(dout), dfinal=dfinal,
                dt_softplus=True, dt_limit=(1e-3, 1e-1))
