"""The two point-wise steps around the scan in the detector's ISSM block, on the library's CUDA kernels:

* `reorder_points(points, index, inverse_index=None)` - the row gather of `Serialization.reorder_points` /
  `reversed_reorder_points` (models/dest_module.py:378-397): `points.gather(dim=1, index=tile(index[..., None]))`
  without materialising the tiled index;
* `PointLiteConv` (models/dest_module.py:400-423) - depthwise Conv1d(k=7, padding=3, groups=C) + SiLU over a
  channels-last (B, N, C) tensor, without the two transposes; same constructor, same parameter names
  (`dwconv.weight`, `dwconv.bias`), so a reference state_dict loads unchanged.

Both require the built CUDA library; there is no fallback."""
import ctypes as ct

import torch
from torch import nn

from . import _lib


def _empty(shape, dtype, device):
    """Every output and workspace of this module is allocated here (the guard-band tests substitute it)."""
    return torch.empty(tuple(shape), dtype=dtype, device=device)


def _gather_rows(src, index):
    if not src.is_cuda:
        raise RuntimeError("dest3d_b200.pointops runs on CUDA tensors only")
    if src.dim() != 3 or index.dim() != 2 or index.shape[0] != src.shape[0]:
        raise ValueError("points must be (B, N, C) and index (B, M)")
    if src.stride(2) != 1:
        src = src.contiguous()
    index = index.to(torch.int64).contiguous()
    B, N, Cc = src.shape
    M = index.shape[1]
    dst = _empty((B, M, Cc), src.dtype, src.device)
    status = torch.zeros(1, dtype=torch.int32, device=src.device)
    if dst.numel() == 0:
        return dst, status
    if N == 0:
        raise IndexError("reorder_points: gather from an empty point set")
    es = src.element_size()
    if (Cc * es) % 2:
        raise ValueError("rows must be an even number of bytes")
    with torch.cuda.device(src.device):
        rc = _lib.lib().issm_b200_gather_rows(src.data_ptr(), index.data_ptr(), dst.data_ptr(), B, M, N, Cc * es,
                                              src.stride(0) * es, src.stride(1) * es, status.data_ptr(),
                                              _lib.stream_ptr(src.device))
    if rc:
        raise _lib.IssmError(rc, "issm_b200_gather_rows")
    return dst, status


class _ReorderFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, points, index, inverse_index, check):
        out, status = _gather_rows(points, index)
        if check and int(status.item()) != 0:
            raise IndexError("reorder_points: index out of range")
        ctx.save_for_backward(index, inverse_index)
        ctx.n_src = points.shape[1]
        return out

    @staticmethod
    def backward(ctx, dout):
        index, inverse_index = ctx.saved_tensors
        if inverse_index is not None:                      # a permutation: the adjoint is the inverse gather
            return _gather_rows(dout, inverse_index)[0], None, None, None
        dsrc = torch.zeros((dout.shape[0], ctx.n_src, dout.shape[2]), dtype=dout.dtype, device=dout.device)
        dsrc.scatter_add_(1, index.unsqueeze(-1).expand(-1, -1, dout.shape[2]), dout)
        return dsrc, None, None, None


def reorder_points(points, index, inverse_index=None, check=False):
    """points (B, N, C), index (B, M) -> (B, M, C) with out[b, i] = points[b, index[b, i]].  When `index` is a
    permutation and `inverse_index` its inverse (the reference keeps both, models/dest_module.py:340-344), the
    backward is one more gather; otherwise it is a scatter-add.  `check=True` synchronises and raises on an index
    outside [0, N) (such rows are left unwritten)."""
    return _ReorderFn.apply(points, index, inverse_index, check)


def _conv_params(x, wf, bf):
    p = _lib.IssmConvParams()
    p.batch, p.seqlen, p.channels = x.shape
    p.io_dtype = _lib.dtype_code(x.dtype)
    p.x, p.x_sb, p.x_sl = x.data_ptr(), x.stride(0), x.stride(1)
    p.weight, p.bias = wf.data_ptr(), _lib.ptr(bf)
    return p


class DwConv7SiluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias):
        if not x.is_cuda:
            raise RuntimeError("dest3d_b200.pointops runs on CUDA tensors only")
        if x.dim() != 3 or weight.shape != (x.shape[2], 1, 7):
            raise ValueError("x must be (B, N, C) and weight (C, 1, 7)")
        if x.stride(2) != 1:
            x = x.contiguous()
        wf = weight.detach().reshape(-1, 7).float().contiguous()
        bf = None if bias is None else bias.detach().float().contiguous()
        y = _empty(x.shape, x.dtype, x.device)
        if y.numel():
            p = _conv_params(x, wf, bf)
            p.y = y.data_ptr()
            with torch.cuda.device(x.device):
                rc = _lib.lib().issm_b200_dwconv7_silu_fwd(ct.byref(p), _lib.stream_ptr(x.device))
            if rc:
                raise _lib.IssmError(rc, "issm_b200_dwconv7_silu_fwd")
        ctx.save_for_backward(x, weight, bias)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, weight, bias = ctx.saved_tensors
        if dy.stride(2) != 1:
            dy = dy.contiguous()
        dy = dy.to(x.dtype)
        wf = weight.detach().reshape(-1, 7).float().contiguous()
        bf = None if bias is None else bias.detach().float().contiguous()
        dx = _empty(x.shape, x.dtype, x.device)
        dw = _empty(wf.shape, torch.float32, x.device)
        db = None if bias is None else _empty(bias.shape, torch.float32, x.device)
        if not x.numel():
            dw.zero_()
            if db is not None:
                db.zero_()
        else:
            p = _conv_params(x, wf, bf)
            p.dy, p.dy_sb, p.dy_sl = dy.data_ptr(), dy.stride(0), dy.stride(1)
            p.dx, p.dweight, p.dbias = dx.data_ptr(), dw.data_ptr(), _lib.ptr(db)
            need = _lib.lib().issm_b200_dwconv_workspace_bytes(ct.byref(p))
            ws = _empty((need,), torch.uint8, x.device)
            p.workspace, p.workspace_bytes = ws.data_ptr(), need
            with torch.cuda.device(x.device):
                rc = _lib.lib().issm_b200_dwconv7_silu_bwd(ct.byref(p), _lib.stream_ptr(x.device))
            if rc:
                raise _lib.IssmError(rc, "issm_b200_dwconv7_silu_bwd")
        return dx, dw.reshape(weight.shape).to(weight.dtype), None if db is None else db.to(bias.dtype)


class PointLiteConv(nn.Module):
    """Drop-in for the reference's PointLiteConv (models/dest_module.py:400-423)."""

    def __init__(self, in_channels: int, out_channels: int):
        super().__init__()
        if in_channels != out_channels:
            raise ValueError("the depthwise convolution needs in_channels == out_channels (groups = out_channels)")
        self.dwconv = nn.Conv1d(in_channels, out_channels, kernel_size=7, stride=1, padding=3, bias=True, groups=out_channels)
        self.act = nn.SiLU()                               # kept for module-tree parity; fused into the kernel

    def forward(self, xyz, feature):
        """xyz (B, N, 3) is unused, as in the reference; feature (B, N, C) -> (B, N, C)."""
        return DwConv7SiluFn.apply(feature, self.dwconv.weight, self.dwconv.bias)
