"""CPU restatement of the steps either side of the scan in the detector's ISSM block.  TEST INFRASTRUCTURE ONLY: the
checker for the CUDA kernels in dest3d_b200/csrc/issm_pointops.cu and issm_glue.cu; the product never imports it.

Pinned: `tests/golden/pointops_golden.npz` holds inputs and outputs of the reference's own classes and of its own
`MultiHeadISSMScan.forward` (captured at the call of the scan), produced by `tests/golden/make_golden_pointops.py`;
`tests/test_oracle_cpu.py` checks every function below against them.

Everything is written with explicit index arithmetic (no convolution or gather library call), in the dtype of the
inputs (use float64), and is differentiable with torch autograd."""
import torch


def reorder_points(points, index):
    """out[b, i, :] = points[b, index[b, i], :].
    Reference: Serialization.reorder_points / reversed_reorder_points, models/dest_module.py:378-397
    (`points.gather(dim=1, index=tile(index[..., None], (1, 1, C)))`)."""
    B = points.shape[0]
    return torch.stack([points[b][index[b]] for b in range(B)], dim=0)


def point_lite_conv(feature, weight, bias):
    """feature (B, N, C), weight (C, 1, 7), bias (C) -> (B, N, C):
        y[b, n, c] = silu(bias[c] + sum_k weight[c, 0, k] * feature[b, n + k - 3, c]),   zero outside [0, N).
    Reference: PointLiteConv, models/dest_module.py:400-423 (Conv1d(C, C, 7, padding=3, groups=C) on the transposed
    tensor, then SiLU, transposed back)."""
    B, N, C = feature.shape
    pad = torch.zeros(B, 3, C, dtype=feature.dtype)
    xp = torch.cat([pad, feature, pad], dim=1)
    pre = bias.to(feature.dtype).reshape(1, 1, C).expand(B, N, C)
    for k in range(7):
        pre = pre + xp[:, k:k + N, :] * weight[:, 0, k].to(feature.dtype).reshape(1, 1, C)
    return pre * torch.sigmoid(pre)


def softplus20(v):
    """torch.nn.functional.softplus with its default threshold 20 (what models/dest_module.py:553 calls)."""
    return torch.where(v > 20.0, v, torch.log1p(torch.exp(torch.clamp(v, max=20.0))))


def adaptive_dt_bc(dist, w_dt, w_bc, dt_tok, dt_bias, b_bias, c_bias, b_bias_back=None, c_bias_back=None, mask=None):
    """dt, B, C (and the second direction's B, C) as MultiHeadISSMScan.forward builds them, models/dest_module.py:541-559:
        bc = bc_proj(dist); b_base, c_base = split(bc);  B = b_base^T + b_bias[..., None];  C alike        (:543-547)
        B_back = b_base^T + b_bias_back[..., None];  C_back alike                                            (:549-551)
        dt = softplus(dt_proj(dist)^T + dt_tok[..., None] + dt_bias[None, None, :, None])                  (:552-553)
        dt = dt * mask[:, :, None]  (float mask)   or   dt[mask] = 0  (bool mask)                          (:555-559)
    dist (b, L, K, M); w_dt (H, M); w_bc (2 G, M); dt_tok (b, L, H); dt_bias (H); b_bias, c_bias (b, L, G); mask (b, L, K).
    Returns (dt (b, L, H, K), B (b, L, G, K), C[, B_back, C_back])."""
    G = w_bc.shape[0] // 2
    proj = lambda w: torch.einsum("blkm,rm->blrk", dist, w.to(dist.dtype))       # Linear without bias, already transposed
    bc = proj(w_bc)
    b_base, c_base = bc[:, :, :G], bc[:, :, G:]
    out = [None, b_base + b_bias.to(dist.dtype).unsqueeze(-1), c_base + c_bias.to(dist.dtype).unsqueeze(-1)]
    if b_bias_back is not None:
        out += [b_base + b_bias_back.to(dist.dtype).unsqueeze(-1), c_base + c_bias_back.to(dist.dtype).unsqueeze(-1)]
    dt = softplus20(proj(w_dt) + dt_tok.to(dist.dtype).unsqueeze(-1) + dt_bias.to(dist.dtype).reshape(1, 1, -1, 1))
    if mask is not None:
        if mask.dtype == torch.bool:
            dt = torch.where(mask.unsqueeze(2), torch.zeros((), dtype=dt.dtype), dt)
        else:
            dt = dt * mask.to(dt.dtype).unsqueeze(2)
    out[0] = dt
    return tuple(out)
