"""dt, B and C of the scan from the query-to-point distance features, as `MultiHeadISSMScan.forward` builds them
(models/dest_module.py:541-559), in one fused pass over `dist` instead of two Linear layers, two transposes and four
elementwise passes:

    bc = bc_proj(dist);  B = b_base^T + b_bias[..., None];  C = c_base^T + c_bias[..., None]   (and the *_back pair)
    dt = softplus(dt_proj(dist)^T + dt_bias_tok[..., None] + dt_bias[None, None, :, None]);  dt = dt * mask[:, :, None]

`adaptive_dt_bc` returns them in the layouts the scan takes: dt (b, L, H, K), B / C (b, L, G, K) (views of one buffer).
Requires the built CUDA library; there is no fallback."""
import ctypes as ct

import torch

from . import _lib


def _empty(shape, dtype, device):
    """Every output and workspace of this module is allocated here (the guard-band tests substitute it)."""
    return torch.empty(tuple(shape), dtype=dtype, device=device)


def _params(dist, w, tok, mask, H, G, back, out_dtype):
    p = _lib.IssmGlueParams()
    p.batch, p.seqlen, p.nstates, p.nfeat = dist.shape
    p.nheads, p.ngroups, p.has_back = H, G, int(back)
    p.io_dtype, p.dist_dtype = _lib.dtype_code(out_dtype), _lib.dtype_code(dist.dtype)
    p.dist, p.dist_sb, p.dist_sl, p.dist_sk = dist.data_ptr(), dist.stride(0), dist.stride(1), dist.stride(2)
    p.weight, p.tok, p.mask = w.data_ptr(), tok.data_ptr(), _lib.ptr(mask)
    return p


class AdaptiveDtBcFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, dist, w_dt, w_bc, tok, mask, H, G, back, out_dtype):
        if not dist.is_cuda:
            raise RuntimeError("dest3d_b200.adaptive_params runs on CUDA tensors only")
        if dist.stride(3) != 1:
            dist = dist.contiguous()
        b, L, K, M = dist.shape
        w = torch.cat([w_dt.detach().float(), w_bc.detach().float()], dim=0).contiguous()
        tokf = tok.detach().float().contiguous()
        maskf = None if mask is None else mask.float().contiguous()
        nb = (4 if back else 2) * G
        if out_dtype != dist.dtype and not (dist.dtype == torch.float32 and out_dtype == torch.bfloat16):
            raise TypeError("adaptive_dt_bc: outputs take the dtype of dist, or bfloat16 next to a float32 dist")
        dt = _empty((b, L, H, K), out_dtype, dist.device)
        bc = _empty((b, L, nb, K), out_dtype, dist.device)
        p = _params(dist, w, tokf, maskf, H, G, back, out_dtype)
        p.dt, p.bc = dt.data_ptr(), bc.data_ptr()
        with torch.cuda.device(dist.device):
            rc = _lib.lib().issm_b200_glue_fwd(ct.byref(p), _lib.stream_ptr(dist.device))
        if rc:
            raise _lib.IssmError(rc, "issm_b200_glue_fwd")
        ctx.save_for_backward(dist, w, tokf, maskf)
        ctx.meta = (H, G, back, w_dt.dtype, w_bc.dtype, tok.dtype, out_dtype)
        # B, C (and the second direction's) go out as separate views of the one buffer, so that their gradients come back
        # one by one and are joined by ONE concatenation (slicing a single output would cost a zero fill and an add each)
        return (dt,) + tuple(bc[:, :, i * G:(i + 1) * G] for i in range(nb // G))

    @staticmethod
    def backward(ctx, ddt, *dparts):
        dist, w, tokf, maskf = ctx.saved_tensors
        dbc = None
        if any(g is not None for g in dparts):
            shape = next(g for g in dparts if g is not None).shape
            dbc = torch.cat([g if g is not None else torch.zeros(shape, dtype=ctx.meta[6], device=dist.device) for g in
                             (gg if gg is None else gg.to(ctx.meta[6]) for gg in dparts)], dim=2)
        H, G, back, wdt_t, wbc_t, tok_t, out_dtype = ctx.meta
        b, L, K, M = dist.shape
        RW = H + 2 * G
        ddist = _empty((b, L, K, M), dist.dtype, dist.device)
        dw = _empty((RW, M), torch.float32, dist.device)
        dtok = _empty(tokf.shape, torch.float32, dist.device)
        p = _params(dist, w, tokf, maskf, H, G, back, out_dtype)
        keep = []
        for name, g in (("ddt", ddt), ("dbc", dbc)):
            if g is not None:
                g = g.to(out_dtype).contiguous()
                keep.append(g)
                setattr(p, name, g.data_ptr())
        p.ddist, p.dweight, p.dtok = ddist.data_ptr(), dw.data_ptr(), dtok.data_ptr()
        need = _lib.lib().issm_b200_glue_workspace_bytes(ct.byref(p))
        ws = _empty((need,), torch.uint8, dist.device)
        p.workspace, p.workspace_bytes = ws.data_ptr(), need
        with torch.cuda.device(dist.device):
            rc = _lib.lib().issm_b200_glue_bwd(ct.byref(p), _lib.stream_ptr(dist.device))
        if rc:
            raise _lib.IssmError(rc, "issm_b200_glue_bwd")
        return ddist, dw[:H].to(wdt_t), dw[H:].to(wbc_t), dtok.to(tok_t), None, None, None, None, None


def adaptive_dt_bc(dist, dt_proj_weight, bc_proj_weight, dt_bias_tok, dt_bias, b_bias, c_bias, b_bias_back=None,
                   c_bias_back=None, mask=None, out_dtype=None):
    """dist (b, L, K, M); dt_proj_weight (H, M); bc_proj_weight (2 G, M); dt_bias_tok (b, L, H) and the parameter dt_bias
    (H,); b_bias / c_bias (b, L, G) (and the second direction's).  `mask` (b, L, K): a float mask multiplies dt, a bool
    mask zeroes dt where it is True (models/dest_module.py:554-558).  `out_dtype`: dtype of dt / B / C (default: that of dist;
    bfloat16 next to a float32 dist is what autocast calls for, without a cast pass over dist).  Returns (dt, B, C) or (dt, B, C, B_back, C_back)."""
    H, G = dt_proj_weight.shape[0], bc_proj_weight.shape[0] // 2
    back = b_bias_back is not None
    terms = [dt_bias_tok.float() + dt_bias.float(), b_bias.float(), c_bias.float()]
    if back:
        terms += [b_bias_back.float(), c_bias_back.float()]
    tok = torch.cat(terms, dim=-1)
    if mask is not None and mask.dtype == torch.bool:
        mask = (~mask).float()
    return AdaptiveDtBcFn.apply(dist, dt_proj_weight, bc_proj_weight, tok, mask, H, G, back, out_dtype or dist.dtype)
