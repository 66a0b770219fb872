"""Drop-in demonstration: the reference's own caller, `MultiHeadISSMScan` (models/dest_module.py:425-612), imported
UNMODIFIED from the copy under baseline/_ref and run on the GPU with the import shim `dest3d_b200/shim` ahead of
it on sys.path, so that its two imports (models/dest_module.py:12-13) resolve to this library.  The same module
class is then run on the CPU in float64 with the oracle in place of the scan and of the gated norm; outputs and
every parameter gradient must agree.  `timm` is not installed on the test machines; the one name the file
imports from it (DropPath, unused by this module) is stubbed."""
import importlib
import os
import sys
import types

import pytest
import torch

from oracle import issm_oracle as O
from tests import parity

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")
SHIM = os.path.join(ROOT, "dest3d_b200", "shim")


@pytest.fixture()
def dest_module():
    if not os.path.isfile(os.path.join(REF, "models", "dest_module.py")):
        pytest.skip("no copy of the reference under baseline/_ref (see oracle/install_reference.py)")
    saved_path, saved_mods = list(sys.path), dict(sys.modules)
    for name in [m for m in sys.modules if m.split(".")[0] in ("issm_triton", "models", "timm")]:
        del sys.modules[name]
    timm, tm, tl = types.ModuleType("timm"), types.ModuleType("timm.models"), types.ModuleType("timm.models.layers")
    tl.DropPath = torch.nn.Identity
    timm.models, tm.layers = tm, tl
    sys.modules.update({"timm": timm, "timm.models": tm, "timm.models.layers": tl})
    sys.path[:0] = [SHIM, REF]
    try:
        dm = importlib.import_module("models.dest_module")
        import dest3d_b200
        assert dm.ISSM_chunk_scan_combined is dest3d_b200.ISSM_chunk_scan_combined      # the shim won the import
        assert dm.RMSNormGated is dest3d_b200.RMSNorm
        yield dm
    finally:
        sys.path[:] = saved_path
        for name in [m for m in sys.modules if m not in saved_mods]:
            del sys.modules[name]


class OracleGatedRMSNorm(torch.nn.Module):
    """The reference's `rms_norm_ref` arithmetic (layernorm_gated.py:8-29) in the parameters' dtype."""

    def __init__(self, hidden, eps=1e-5, norm_before_gate=False):
        super().__init__()
        self.eps, self.nbg = eps, norm_before_gate
        self.weight = torch.nn.Parameter(torch.ones(hidden))

    def forward(self, x, z=None):
        if z is not None and not self.nbg:
            x = x * torch.nn.functional.silu(z)
        y = x * torch.rsqrt(x.square().mean(-1, keepdim=True) + self.eps) * self.weight
        if z is not None and self.nbg:
            y = y * torch.nn.functional.silu(z)
        return y


def oracle_scan(x, dt, A, B, C, chunk_size, D=None, z=None, dt_bias=None, initial_states=None, seq_idx=None,
                dt_softplus=False, dt_limit=(0.0, float("inf")), return_final_states=False):
    out, fin = O.issm_scan_chunked(x, dt, A, B, C, 64, D=D, z=z, dt_bias=dt_bias, initial_states=initial_states,
                                   dt_softplus=dt_softplus, dt_limit=dt_limit, compute_dtype=torch.float64)
    return (out, fin) if return_final_states else out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16_autocast"])
def test_reference_caller_through_the_shim(dest_module, dtype):
    """float32: parameters and activations in float32 (fp32 kernels), nominal float32 tolerance.  bfloat16: the
    float32 module under torch.autocast, as the detector is trained: x, B, C, z and the initial states reach the
    scan in bfloat16 and dt in float32 (autocast keeps softplus in float32), which is the tensor-core path."""
    dm = dest_module
    torch.manual_seed(0)
    batch, L, K, d_model, d_dist, nheads = 1, 384, 256, 144, 16, 8           # d_inner 288 = 8 heads x 36, 256 query states
    kw = dict(d_model=d_model, d_state=K, d_dist=d_dist, chunk_size=K, nheads=nheads, expand=2, use_biscan=True)
    gpu = dm.MultiHeadISSMScan(**kw)
    with torch.no_grad():                                     # lively decays and non-trivial D / norm weights
        gpu.A_log.copy_(torch.log(torch.rand(nheads) * 15 + 1))
        gpu.D.copy_(torch.randn(nheads))
        gpu.key_norm.weight.copy_(1 + 0.02 * torch.randn(2 * d_model))
        gpu.dt_proj.weight.mul_(0.2)
    state = {k: v.detach().clone() for k, v in gpu.state_dict().items()}
    in_key, in_query = torch.randn(batch, L, d_model), torch.randn(batch, K, d_model) / 4
    dist, xyz = torch.randn(batch, L, K, d_dist), torch.randn(batch, L, 3)
    mask = (torch.rand(batch, L, K) > 0.1).float()
    gk, gq = torch.randn(batch, L, d_model), torch.randn(batch, K, d_model)

    # CPU, float64: the same module class with the oracle patched in for the scan and the gated norm
    real_scan, real_norm = dm.ISSM_chunk_scan_combined, dm.RMSNormGated
    dm.ISSM_chunk_scan_combined, dm.RMSNormGated = oracle_scan, OracleGatedRMSNorm
    try:
        ref = dm.MultiHeadISSMScan(**kw)
    finally:
        dm.RMSNormGated = real_norm
    ref.load_state_dict(state)
    ref = ref.double()
    cast = lambda t: t.double()
    try:
        ok_ref, oq_ref = ref(cast(in_key), cast(in_query), cast(dist), cast(xyz), mask)   # float32 mask: the multiply branch (dest_module.py:556-557)
        ((ok_ref * gk.double()).sum() + (oq_ref * gq.double()).sum()).backward()
    finally:
        dm.ISSM_chunk_scan_combined = real_scan

    gpu = gpu.cuda()
    c = lambda t: t.cuda()
    torch.backends.cudnn.allow_tf32 = False                  # the module's depthwise convolution, in float32
    torch.backends.cuda.matmul.allow_tf32 = False
    seen = []
    real = dm.ISSM_chunk_scan_combined

    def spy(x, dt, A, B, C, *a, **k):
        seen.append((x.dtype, dt.dtype))
        if dtype == torch.bfloat16:                          # the reference's own tensors must reach the tensor-core kernels
            import ctypes as ct
            from dest3d_b200 import _lib, issm_combined
            p, keep = issm_combined._fill_common(x, dt, A, B, C, k.get("chunk_size", a[0] if a else 256), k.get("D"), None, None,
                                                 k.get("initial_states"), False, (0.0, float("inf")), False, "auto")
            assert _lib.lib().issm_b200_resolve_path_pass(ct.byref(p), 0) == _lib.PATH_TENSOR, (B.stride(), C.stride(), dt.stride())
        return real(x, dt, A, B, C, *a, **k)

    dm.ISSM_chunk_scan_combined = spy
    try:
        with torch.autocast("cuda", dtype=torch.bfloat16, enabled=dtype == torch.bfloat16):
            ok, oq = gpu(c(in_key), c(in_query), c(dist), c(xyz), mask.cuda())     # float32 mask: dt = softplus(...) * mask
        ((ok.float() * gk.cuda()).sum() + (oq.float() * gq.cuda()).sum()).backward()
    finally:
        dm.ISSM_chunk_scan_combined = real
    assert seen == [(dtype, torch.float32)] * 2, seen        # both scan directions, in the expected dtypes
    rep = []
    loosen = 1.0 if dtype == torch.float32 else 4.0           # bf16 linear layers around the scan add their own rounding
    parity.close(ok, ok_ref, dtype, "out_key", rep, loosen, literal=False)
    parity.close(oq, oq_ref, dtype, "out_query", rep, loosen, literal=False)
    ref_grads = dict(ref.named_parameters())
    for name, p in gpu.named_parameters():
        assert p.grad is not None, name
        parity.close(p.grad, ref_grads[name].grad, dtype, "d" + name, rep, loosen, literal=False)
    print("MultiHeadISSMScan through the shim:", parity.format_report(rep))

    # the same block assembled from this library's kernels (fused PointLiteConv, dt / B / C generation, reverse scan
    # without flips): the reference's state_dict loads unchanged, results against the same float64 run
    from dest3d_b200.issm_block import MultiHeadISSMScan as NativeBlock
    mine = NativeBlock(**kw)
    mine.load_state_dict(state)
    mine = mine.cuda()
    with torch.autocast("cuda", dtype=torch.bfloat16, enabled=dtype == torch.bfloat16):
        ok2, oq2 = mine(c(in_key), c(in_query), c(dist), c(xyz), mask.cuda())
    ((ok2.float() * gk.cuda()).sum() + (oq2.float() * gq.cuda()).sum()).backward()
    rep = []
    parity.close(ok2, ok_ref, dtype, "out_key", rep, loosen, literal=False)
    parity.close(oq2, oq_ref, dtype, "out_query", rep, loosen, literal=False)
    for name, p in mine.named_parameters():
        assert p.grad is not None, name
        parity.close(p.grad, ref_grads[name].grad, dtype, "d" + name, rep, loosen, literal=False)
    print("the block on this library's kernels:", parity.format_report(rep))
