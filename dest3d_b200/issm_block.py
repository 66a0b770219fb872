"""`MultiHeadISSMScan` (models/dest_module.py:426-612) assembled from this library's kernels: the reference's
constructor, parameter names (a reference state_dict loads unchanged) and forward signature, with

  * the two PointLiteConv layers on the channels-last kernels (`pointops.PointLiteConv`), no transposes;
  * dt, B, C and the second direction's B, C from `dist` in one fused pass (`adaptive_params.adaptive_dt_bc`) instead of
    dt_proj / bc_proj, the transposes and the elementwise passes of lines 543-558;
  * both scan directions over the same dt without the four flipped copies of lines 567-573 (`reverse=True`);
  * the z-gated RMSNorm kernel.
The dense projections stay `nn.Linear` (library GEMMs)."""
import math

import torch
from torch import nn

from .adaptive_params import adaptive_dt_bc
from .issm_combined import issm_bidirectional_scan, ISSM_chunk_scan_combined
from .layernorm_gated import RMSNorm as RMSNormGated
from .pointops import PointLiteConv


class MultiHeadISSMScan(nn.Module):
    def __init__(self, d_model=512, d_state=64, d_dist=4, chunk_size=256, nheads=4, ngroups=1, expand=2, use_biscan=True,
                 A_init_range=(1, 16), dt_min=0.0001, dt_max=0.1, dt_init_floor=1e-4, dt_limit=(0.0, float("inf")), layer_idx=None):
        super().__init__()
        self.d_model, self.d_state, self.d_dist, self.chunk_size = d_model, d_state, d_dist, chunk_size
        self.nheads, self.ngroups, self.expand, self.use_biscan = nheads, ngroups, expand, use_biscan
        self.d_inner = expand * d_model
        self.headdim = self.d_inner // nheads
        self.dt_limit, self.layer_idx = dt_limit, layer_idx
        # projections (models/dest_module.py:469-482)
        self.key_proj = nn.Linear(d_model, 2 * self.d_inner + 2 * ngroups + nheads, bias=False)
        d_key_conv = self.d_inner + 2 * ngroups
        self.key_conv = PointLiteConv(d_key_conv, d_key_conv)
        if use_biscan:
            self.key_conv_back = PointLiteConv(d_key_conv, d_key_conv)
        self.query_proj = nn.Linear(d_model, self.d_inner, bias=False)
        self.bc_proj = nn.Linear(d_dist, 2 * ngroups, bias=False)
        self.dt_proj = nn.Linear(d_dist, nheads, bias=False)
        # step size and decay parameters (models/dest_module.py:484-508)
        dt = torch.exp(torch.rand(nheads) * (math.log(dt_max) - math.log(dt_min)) + math.log(dt_min)).clamp(min=dt_init_floor)
        self.dt_bias = nn.Parameter(dt + torch.log(-torch.expm1(-dt)))          # inverse of softplus
        self.dt_bias._no_weight_decay = True
        assert A_init_range[0] > 0 and A_init_range[1] >= A_init_range[0]
        self.A_log = nn.Parameter(torch.log(torch.empty(nheads, dtype=torch.float32).uniform_(*A_init_range)))
        self.A_log._no_weight_decay = True
        self.D = nn.Parameter(torch.ones(nheads))
        self.D._no_weight_decay = True
        # output layers (models/dest_module.py:510-517)
        self.out_key_proj = nn.Linear(self.d_inner, d_model, bias=False)
        self.out_query_proj = nn.Linear(self.d_inner, d_model, bias=False)
        self.key_norm = RMSNormGated(self.d_inner, eps=1e-5, norm_before_gate=False)
        self.query_norm = nn.LayerNorm(self.d_inner)

    def forward(self, in_key, in_query, dist, key_xyz, mask=None):
        """in_key (B, L, D), in_query (B, K, D), dist (B, L, K, M), mask (B, L, K) -> out_key (B, L, D), out_query (B, K, D)."""
        G, H, P = self.ngroups, self.nheads, self.headdim
        zxbcdt = self.key_proj(in_key)
        z, xbc, dt_tok = torch.split(zxbcdt, [self.d_inner, self.d_inner + 2 * G, H], dim=-1)
        xbc = self.key_conv(key_xyz, xbc)
        x, b_bias, c_bias = torch.split(xbc, [self.d_inner, G, G], dim=-1)
        back = (None, None, None)
        if self.use_biscan:                                # the second convolution takes the OUTPUT of the first (dest_module.py:534)
            back = torch.split(self.key_conv_back(key_xyz, xbc), [self.d_inner, G, G], dim=-1)
        initial_states = self.query_proj(in_query)
        bsz, K = initial_states.shape[:2]
        initial_states = initial_states.reshape(bsz, K, H, P).permute(0, 2, 3, 1)           # b l (h hd) -> b h hd l
        A = (-torch.exp(self.A_log.float()))[:, None].expand(H, self.d_state)
        # dt, B, C (and the second direction's B, C) in the scan's layouts, in the activations' dtype
        feats = dist if (dist.dtype == x.dtype or (dist.dtype == torch.float32 and x.dtype == torch.bfloat16)) else dist.to(x.dtype)
        outs = adaptive_dt_bc(feats, self.dt_proj.weight, self.bc_proj.weight, dt_tok, self.dt_bias, b_bias, c_bias,
                              back[1], back[2], mask, out_dtype=x.dtype)
        kw = {} if self.dt_limit == (0.0, float("inf")) else dict(dt_limit=self.dt_limit)
        heads = lambda t: t.reshape(t.shape[0], t.shape[1], H, P)
        if self.use_biscan:
            dt, B, C, B_back, C_back = outs
            key, last_states = issm_bidirectional_scan(heads(x.contiguous()), heads(back[0].contiguous()), dt, A, B, C, B_back, C_back,
                                                       self.chunk_size, D=self.D, initial_states=initial_states, **kw)
        else:
            dt, B, C = outs
            key, last_states = ISSM_chunk_scan_combined(heads(x.contiguous()), dt, A, B, C, self.chunk_size, D=self.D,
                                                        initial_states=initial_states, return_final_states=True, **kw)
        key = self.key_norm(key.reshape(key.shape[0], key.shape[1], H * P), z)
        out_key = self.out_key_proj(key)
        last_states = last_states.permute(0, 3, 1, 2).reshape(bsz, K, H * P)                # b h p l -> b l (h p)
        out_query = self.out_query_proj(self.query_norm(last_states.to(out_key.dtype)))
        return out_key, out_query
