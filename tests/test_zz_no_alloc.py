"""The workspace-free backward of the gated norm, for hosts that cannot allocate device memory at
call time (a plugin inside a server with a sealed memory pool, a latency-critical loop, a binding
without a device allocator): called through the C ABI and compared with the regular entry point,
twice in a row because all calls share one built-in scratch array that keeps the previous call's
contents.  Collected last on purpose."""
import ctypes as ct

import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(L, lib_fn, x, z, w, dy, rstd, use_workspace, bias=None, mean=None, out=None):
    """One backward call through the C ABI.  bias / mean given: LayerNorm with bias (the bias-gradient half of the
    partials is used too); else the detector's gated RMSNorm.  `out` = preallocated (dx, dz, dw, db) to write into."""
    from dest3d_b200 import _lib
    rows, hidden = x.shape
    p = _lib.IssmNormParams()
    p.rows, p.hidden, p.group_size = rows, hidden, hidden
    p.io_dtype = _lib.dtype_code(x.dtype)
    p.is_rms, p.norm_before_gate, p.has_z, p.has_bias = int(bias is None), 0, 1, int(bias is not None)
    p.eps = 1e-5
    p.x, p.x_sr, p.z, p.z_sr = x.data_ptr(), x.stride(0), z.data_ptr(), z.stride(0)
    p.weight, p.rstd = w.data_ptr(), rstd.data_ptr()
    if bias is not None:
        p.bias, p.mean = bias.data_ptr(), mean.data_ptr()
    if out is None:
        out = (torch.empty_like(x), torch.empty_like(x), torch.empty(hidden, dtype=torch.float32, device=x.device),
               torch.empty(hidden, dtype=torch.float32, device=x.device))
    dx, dz, dw, db = out
    p.dy, p.dy_sr, p.dx, p.dz, p.dweight = dy.data_ptr(), dy.stride(0), dx.data_ptr(), dz.data_ptr(), dw.data_ptr()
    if bias is not None:
        p.dbias = db.data_ptr()
    ws = None
    if use_workspace:
        need = L.issm_b200_norm_workspace_bytes(ct.byref(p), 1)
        ws = torch.empty(max(int(need), 256), dtype=torch.uint8, device=x.device)
        p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
    rc = lib_fn(ct.byref(p), ct.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, L.issm_b200_strerror(rc)
    torch.cuda.synchronize()
    return (dx, dz, dw, db) if bias is not None else (dx, dz, dw)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_no_alloc_norm_backward_matches_regular_entry_point(dtype):
    from dest3d_b200 import _lib
    L = _lib.lib()
    L.issm_b200_norm_bwd_noalloc.restype = ct.c_int
    L.issm_b200_norm_bwd_noalloc.argtypes = [ct.POINTER(_lib.IssmNormParams), ct.c_void_p]
    rtol, atol = (1e-4, 1e-5) if dtype == torch.float32 else (1e-2, 1e-2)
    for call, (rows, hidden, seed) in enumerate(((3000, 288, 1), (777, 1024, 2))):   # two calls in a row
        g = torch.Generator().manual_seed(seed)
        x = torch.randn(rows, hidden, generator=g).to(dtype).cuda()
        z = torch.randn(rows, hidden, generator=g).to(dtype).cuda()
        dy = torch.randn(rows, hidden, generator=g).to(dtype).cuda()
        w = (1 + 0.02 * torch.randn(hidden, generator=g)).cuda()
        xs = x.float() * torch.nn.functional.silu(z.float())
        rstd = torch.rsqrt(xs.square().mean(-1) + 1e-5).contiguous()
        ref = _run(L, L.issm_b200_norm_bwd, x, z, w, dy, rstd, True)
        before = torch.cuda.memory_allocated()
        got = _run(L, L.issm_b200_norm_bwd_noalloc, x, z, w, dy, rstd, False)
        assert torch.cuda.memory_allocated() - before <= 3 * x.numel() * x.element_size() + 8192   # outputs only
        for name, a, b in zip(("dx", "dz", "dweight"), got, ref):
            scale = max(1.0, b.float().abs().max().item())
            assert torch.allclose(a.float(), b.float(), rtol=rtol, atol=atol * scale), f"call {call}: {name}"


def test_no_alloc_layernorm_with_bias_and_device_memory_unchanged():
    """LayerNorm with bias exercises the bias-gradient half of the built-in scratch.  With every output
    preallocated, the free device memory reported by the driver is the same before and after the second call:
    nothing was allocated behind torch's back either (torch's own counter cannot see a cudaMalloc)."""
    from dest3d_b200 import _lib
    L = _lib.lib()
    L.issm_b200_norm_bwd_noalloc.restype = ct.c_int
    L.issm_b200_norm_bwd_noalloc.argtypes = [ct.POINTER(_lib.IssmNormParams), ct.c_void_p]
    g = torch.Generator().manual_seed(5)
    rows, hidden = 2500, 288
    x, z, dy = (torch.randn(rows, hidden, generator=g).cuda() for _ in range(3))
    w = (1 + 0.02 * torch.randn(hidden, generator=g)).cuda()
    bias = (0.1 * torch.randn(hidden, generator=g)).cuda()
    xs = x * torch.nn.functional.silu(z)
    mean = xs.mean(-1).contiguous()
    rstd = torch.rsqrt((xs - mean[:, None]).square().mean(-1) + 1e-5).contiguous()
    ref = _run(L, L.issm_b200_norm_bwd, x, z, w, dy, rstd, True, bias=bias, mean=mean)
    out = tuple(torch.empty_like(t) for t in ref)
    _run(L, L.issm_b200_norm_bwd_noalloc, x, z, w, dy, rstd, False, bias=bias, mean=mean, out=out)   # first call: set-up
    for t in out:
        t.fill_(float("nan"))
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    got = _run(L, L.issm_b200_norm_bwd_noalloc, x, z, w, dy, rstd, False, bias=bias, mean=mean, out=out)
    assert torch.cuda.mem_get_info()[0] == free_before
    for name, a, b in zip(("dx", "dz", "dweight", "dbias"), got, ref):
        scale = max(1.0, b.abs().max().item())
        assert torch.allclose(a, b, rtol=1e-4, atol=1e-5 * scale), name


def test_no_alloc_rejects_rows_wider_than_the_scratch():
    from dest3d_b200 import _lib
    L = _lib.lib()
    L.issm_b200_norm_bwd_noalloc.restype = ct.c_int
    x = torch.randn(4, 2048, device="cuda")
    p = _lib.IssmNormParams()
    p.rows, p.hidden, p.group_size, p.io_dtype, p.is_rms, p.eps = 4, 2048, 2048, 0, 1, 1e-5
    for f in ("x", "weight", "rstd", "dy", "dx", "dweight"):
        setattr(p, f, x.data_ptr())
    rc = L.issm_b200_norm_bwd_noalloc(ct.byref(p), None)
    assert rc == 9 and b"scratch" in L.issm_b200_strerror(rc)
