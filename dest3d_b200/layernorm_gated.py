"""Gated RMSNorm / LayerNorm with the reference's interface (issm_triton/layernorm_gated.py:328-427)
on top of the B200 C ABI: `RMSNorm`, `LayerNorm`, `rmsnorm_fn`, `layernorm_fn`, `LayerNormFn`.  As for the scan,
the default binding is the torch C++ extension (`torch.ops.issm_b200.norm_fwd / norm_bwd`); with
`issm_combined.BINDING == "ctypes"` the calls go through the ctypes binding instead.
"""
import ctypes as ct

import torch

from . import _ext, _lib, issm_combined


def _norm_params(x2, z2, weight, bias, eps, group_size, norm_before_gate, is_rms_norm):
    rows, hidden = x2.shape
    p = _lib.IssmNormParams()
    p.rows, p.hidden = rows, hidden
    p.group_size = hidden if group_size is None else int(group_size)
    assert hidden % p.group_size == 0
    p.io_dtype = _lib.dtype_code(x2.dtype)
    p.is_rms, p.norm_before_gate = int(is_rms_norm), int(norm_before_gate)
    p.has_z, p.has_bias = int(z2 is not None), int(bias is not None)
    p.eps = float(eps)
    p.x, p.x_sr = x2.data_ptr(), x2.stride(0)
    if z2 is not None:
        p.z, p.z_sr = z2.data_ptr(), z2.stride(0)
    p.weight, p.bias = weight.data_ptr(), _lib.ptr(bias)
    return p


class LayerNormFn(torch.autograd.Function):

    @staticmethod
    def forward(ctx, x, weight, bias, z=None, eps=1e-6, group_size=None, norm_before_gate=True,
                is_rms_norm=False):
        """If z is not None, we do norm(x) * silu(z) if norm_before_gate, else norm(x * silu(z))"""
        if not x.is_cuda:
            raise RuntimeError("the gated norm runs on CUDA tensors only; there is no CPU path")
        x_shape_og = x.shape
        x2 = x.reshape(-1, x.shape[-1])
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        z2 = None
        if z is not None:
            assert z.shape == x_shape_og
            z2 = z.reshape(-1, z.shape[-1])
            if z2.dtype != x2.dtype:
                z2 = z2.to(x2.dtype)
            if z2.stride(-1) != 1:
                z2 = z2.contiguous()
        wf = weight.detach().float().contiguous()
        bf = bias.detach().float().contiguous() if bias is not None else None
        if issm_combined.BINDING == "torch":
            y, rstd, mean = _ext.ops().norm_fwd(x2, z2, wf, bf, float(eps), int(group_size or 0), bool(norm_before_gate),
                                                bool(is_rms_norm))
            mean = _ext.opt(mean)
            ctx.save_for_backward(x2, weight, bias, mean, rstd, z2)
            ctx.x_shape_og, ctx.eps, ctx.group_size = x_shape_og, eps, group_size
            ctx.norm_before_gate, ctx.is_rms_norm = norm_before_gate, is_rms_norm
            ctx.z_dtype = None if z is None else z.dtype
            return y.reshape(x_shape_og)
        p = _norm_params(x2, z2, wf, bf, eps, group_size, norm_before_gate, is_rms_norm)
        ng = p.hidden // p.group_size
        y = torch.empty(x2.shape, dtype=x2.dtype, device=x2.device)
        rstd = torch.empty(p.rows * ng, dtype=torch.float32, device=x2.device)
        mean = torch.empty(p.rows * ng, dtype=torch.float32, device=x2.device) if not is_rms_norm else None
        p.y, p.y_sr, p.rstd, p.mean = y.data_ptr(), y.stride(0), rstd.data_ptr(), _lib.ptr(mean)
        with torch.cuda.device(x2.device):
            rc = _lib.lib().issm_b200_norm_fwd(ct.byref(p), _lib.stream_ptr(x2.device))
        if rc:
            raise _lib.IssmError(rc, "issm_b200_norm_fwd")
        ctx.save_for_backward(x2, weight, bias, mean, rstd, z2)
        ctx.x_shape_og = x_shape_og
        ctx.eps = eps
        ctx.group_size = group_size
        ctx.norm_before_gate = norm_before_gate
        ctx.is_rms_norm = is_rms_norm
        ctx.z_dtype = None if z is None else z.dtype
        return y.reshape(x_shape_og)

    @staticmethod
    def backward(ctx, dy):
        x2, weight, bias, mean, rstd, z2 = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if dy2.dtype != x2.dtype:
            dy2 = dy2.to(x2.dtype)
        if dy2.stride(-1) != 1:
            dy2 = dy2.contiguous()
        assert dy2.shape == x2.shape
        wf = weight.detach().float().contiguous()
        bf = bias.detach().float().contiguous() if bias is not None else None
        if issm_combined.BINDING == "torch":
            dx, dz, dw, db = _ext.ops().norm_bwd(dy2, x2, z2, wf, bf, rstd, mean, float(ctx.eps), int(ctx.group_size or 0),
                                                 bool(ctx.norm_before_gate), bool(ctx.is_rms_norm))
            dzo = None
            if z2 is not None:
                dzo = dz.reshape(ctx.x_shape_og)
                if dzo.dtype != ctx.z_dtype:
                    dzo = dzo.to(ctx.z_dtype)
            return (dx.reshape(ctx.x_shape_og), dw.to(weight.dtype), db.to(bias.dtype) if bias is not None else None,
                    dzo, None, None, None, None)
        p = _norm_params(x2, z2, wf, bf, ctx.eps, ctx.group_size, ctx.norm_before_gate, ctx.is_rms_norm)
        dev = x2.device
        dx = torch.empty(x2.shape, dtype=x2.dtype, device=dev)
        dz = torch.empty(x2.shape, dtype=x2.dtype, device=dev) if z2 is not None else None
        dw = torch.empty(p.hidden, dtype=torch.float32, device=dev)
        db = torch.empty(p.hidden, dtype=torch.float32, device=dev) if bias is not None else None
        p.rstd, p.mean = rstd.data_ptr(), _lib.ptr(mean)
        p.dy, p.dy_sr = dy2.data_ptr(), dy2.stride(0)
        p.dx, p.dz, p.dweight, p.dbias = dx.data_ptr(), _lib.ptr(dz), dw.data_ptr(), _lib.ptr(db)
        need = _lib.lib().issm_b200_norm_workspace_bytes(ct.byref(p), 1)
        ws = torch.empty(max(int(need), 256), dtype=torch.uint8, device=dev)
        p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
        with torch.cuda.device(dev):
            rc = _lib.lib().issm_b200_norm_bwd(ct.byref(p), _lib.stream_ptr(dev))
        if rc:
            raise _lib.IssmError(rc, "issm_b200_norm_bwd")
        dzo = None
        if dz is not None:
            dzo = dz.reshape(ctx.x_shape_og)
            if dzo.dtype != ctx.z_dtype:
                dzo = dzo.to(ctx.z_dtype)
        return (dx.reshape(ctx.x_shape_og), dw.to(weight.dtype), db.to(bias.dtype) if db is not None else None,
                dzo, None, None, None, None)


def layernorm_fn(x, weight, bias, z=None, eps=1e-6, group_size=None, norm_before_gate=True, is_rms_norm=False):
    return LayerNormFn.apply(x, weight, bias, z, eps, group_size, norm_before_gate, is_rms_norm)


def rmsnorm_fn(x, weight, bias, z=None, eps=1e-6, group_size=None, norm_before_gate=True):
    return LayerNormFn.apply(x, weight, bias, z, eps, group_size, norm_before_gate, True)


class LayerNorm(torch.nn.Module):

    def __init__(self, hidden_size, eps=1e-5, group_size=None, norm_before_gate=True, device=None, dtype=None):
        """If group_size is not None, we do GroupNorm with each group having group_size elements.
        group_size=None is equivalent to group_size=hidden_size (i.e. there's only 1 group)."""
        factory_kwargs = {"device": device, "dtype": dtype}
        super().__init__()
        self.eps = eps
        self.weight = torch.nn.Parameter(torch.empty(hidden_size, **factory_kwargs))
        self.bias = torch.nn.Parameter(torch.empty(hidden_size, **factory_kwargs))
        self.group_size = group_size
        self.norm_before_gate = norm_before_gate
        self.reset_parameters()

    def reset_parameters(self):
        torch.nn.init.ones_(self.weight)
        torch.nn.init.zeros_(self.bias)

    def forward(self, x, z=None):
        """If z is not None, we do norm(x) * silu(z) if norm_before_gate, else norm(x * silu(z))"""
        return layernorm_fn(x, self.weight, self.bias, z=z, group_size=self.group_size, eps=self.eps,
                            norm_before_gate=self.norm_before_gate)


class RMSNorm(torch.nn.Module):

    def __init__(self, hidden_size, eps=1e-5, group_size=None, norm_before_gate=True, device=None, dtype=None):
        """If group_size is not None, we do GroupNorm with each group having group_size elements.
        group_size=None is equivalent to group_size=hidden_size (i.e. there's only 1 group)."""
        factory_kwargs = {"device": device, "dtype": dtype}
        super().__init__()
        self.eps = eps
        self.weight = torch.nn.Parameter(torch.empty(hidden_size, **factory_kwargs))
        self.register_parameter("bias", None)
        self.group_size = group_size
        self.norm_before_gate = norm_before_gate
        self.reset_parameters()

    def reset_parameters(self):
        torch.nn.init.ones_(self.weight)

    def forward(self, x, z=None):
        """If z is not None, we do norm(x) * silu(z) if norm_before_gate, else norm(x * silu(z))"""
        return rmsnorm_fn(x, self.weight, self.bias, z=z, eps=self.eps, group_size=self.group_size,
                          norm_before_gate=self.norm_before_gate)
