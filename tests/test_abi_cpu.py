"""The C-ABI library builds, loads and exports every symbol the header declares; host-side
argument validation works without a device (no compute call is made here)."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    names = []
    for fn in sorted(os.listdir(os.path.join(ROOT, "include"))):
        if fn.endswith(".h"):
            src = open(os.path.join(ROOT, "include", fn)).read()
            src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
            names += re.findall(r"\b(issm_b200_\w+)\s*\(", src)
    return sorted(set(names))


def test_header_symbols_exported(built_lib):
    names = declared_functions()
    assert len(names) >= 12
    for n in names:
        assert hasattr(built_lib, n), f"{n} declared in include/ but not exported by libissm_b200.so"


def test_struct_layout_matches(built_lib):
    from dest3d_b200 import _lib
    assert built_lib.issm_b200_sizeof_params() == C.sizeof(_lib.IssmParams)
    assert built_lib.issm_b200_sizeof_norm_params() == C.sizeof(_lib.IssmNormParams)
    assert built_lib.issm_b200_version() == 1


def _params(**over):
    from dest3d_b200 import _lib
    p = _lib.IssmParams()
    p.batch, p.seqlen, p.nheads, p.headdim, p.dstate, p.ngroups, p.chunk_size = 2, 100, 4, 36, 64, 1, 64
    p.io_dtype, p.dt_dtype, p.path = _lib.F32, _lib.F32, _lib.PATH_SIMT
    p.dt_min, p.dt_max = 0.0, 3e38
    for k, v in over.items():
        setattr(p, k, v)
    return p


def test_validation_codes_without_device(built_lib):
    L = built_lib
    assert L.issm_b200_fwd(None, None) == 1                                   # ISSM_ERR_NULL
    assert L.issm_b200_fwd(C.byref(_params(seqlen=0)), None) == 2             # ISSM_ERR_SHAPE
    assert L.issm_b200_fwd(C.byref(_params(ngroups=3)), None) == 2
    assert L.issm_b200_fwd(C.byref(_params(chunk_size=512)), None) == 2
    assert L.issm_b200_fwd(C.byref(_params(io_dtype=7)), None) == 3           # ISSM_ERR_DTYPE
    assert L.issm_b200_fwd(C.byref(_params()), None) == 1                     # pointers are null
    assert L.issm_b200_bwd(C.byref(_params()), None) == 1
    assert b"workspace" in L.issm_b200_strerror(4)


def test_workspace_query(built_lib):
    L = built_lib
    fwd = L.issm_b200_workspace_bytes(C.byref(_params()), 0)
    bwd = L.issm_b200_workspace_bytes(C.byref(_params()), 1)
    assert 0 < fwd < bwd
    assert fwd % 256 == 0
    assert L.issm_b200_workspace_bytes(C.byref(_params(seqlen=-1)), 0) == 0
    # fp32 activations never take the tensor-core path
    assert L.issm_b200_resolve_path(C.byref(_params(path=0))) == 1


def test_workspace_too_small_is_reported(built_lib):
    """Pointers set to a dummy non-null value; the call must stop at the workspace check,
    before anything would be launched."""
    L = built_lib
    p = _params()
    for f in ("x", "dt", "A", "B", "C", "out"):
        setattr(p, f, 256)
    p.workspace, p.workspace_bytes = 256, 16
    assert L.issm_b200_fwd(C.byref(p), None) == 4                             # ISSM_ERR_WORKSPACE


def test_misaligned_tensor_path_buffers_are_reported(built_lib):
    """saved_states, dB and dC of the tensor-core path are accessed 16 bytes at a time; a caller that passes a
    sub-view at an 8-byte offset gets ISSM_ERR_ALIGN before anything is launched (dummy pointers, no device)."""
    from dest3d_b200 import _lib
    L = built_lib
    p = _params(io_dtype=_lib.BF16, dt_dtype=_lib.BF16, path=_lib.PATH_TENSOR, dstate=256, chunk_size=256)
    p.x_sb, p.x_sl, p.x_sh = 100 * 4 * 36, 4 * 36, 36
    p.out_sb, p.out_sl, p.out_sh = p.x_sb, p.x_sl, p.x_sh
    p.dout_sb, p.dout_sl, p.dout_sh = p.x_sb, p.x_sl, p.x_sh
    p.dt_sb, p.dt_sl, p.dt_sh = 100 * 4 * 256, 4 * 256, 256
    p.B_sb, p.B_sl, p.B_sg = 100 * 256, 256, 256
    p.C_sb, p.C_sl, p.C_sg = 100 * 256, 256, 256
    for f in ("x", "dt", "A", "B", "C", "out", "dout", "dx", "ddt", "dB", "dC", "dA"):
        setattr(p, f, 4096)
    assert L.issm_b200_resolve_path(C.byref(p)) == _lib.PATH_TENSOR
    need = L.issm_b200_workspace_bytes(C.byref(p), 1)
    assert need > 0
    p.workspace, p.workspace_bytes = 1 << 20, need
    p.saved_states = 4096 + 8
    assert L.issm_b200_fwd(C.byref(p), None) == 5                             # ISSM_ERR_ALIGN
    assert L.issm_b200_bwd(C.byref(p), None) == 5
    p.saved_states = 4096
    p.dB = 4096 + 8
    assert L.issm_b200_bwd(C.byref(p), None) == 5
    p.dB, p.dC = 4096, 4096 + 2
    assert L.issm_b200_bwd(C.byref(p), None) == 5


def test_norm_validation(built_lib):
    from dest3d_b200 import _lib
    p = _lib.IssmNormParams()
    p.rows, p.hidden, p.group_size = 4, 288, 100
    assert built_lib.issm_b200_norm_fwd(C.byref(p), None) == 2                # group does not divide hidden
    p.group_size = 288
    assert built_lib.issm_b200_norm_fwd(C.byref(p), None) == 1                # null pointers


def test_operators_refuse_cpu_tensors(built_lib):
    import torch
    from dest3d_b200 import RMSNorm
    with pytest.raises(RuntimeError):
        RMSNorm(16)(torch.randn(2, 16))


def test_point_ops_validation(built_lib):
    """Serialization gather and PointLiteConv entry points: struct layout and the codes returned before any launch."""
    import torch
    from dest3d_b200 import PointLiteConv, _lib, reorder_points
    L = _lib.lib()
    assert L.issm_b200_sizeof_conv_params() == C.sizeof(_lib.IssmConvParams)
    p = _lib.IssmConvParams()
    assert L.issm_b200_dwconv7_silu_fwd(None, None) == 1
    assert L.issm_b200_dwconv7_silu_fwd(C.byref(p), None) == 2                # zero sizes
    p.batch, p.seqlen, p.channels = 2, 100, 290
    assert L.issm_b200_dwconv7_silu_fwd(C.byref(p), None) == 1                # null pointers
    p.io_dtype = 9
    assert L.issm_b200_dwconv7_silu_fwd(C.byref(p), None) == 3
    p.io_dtype = _lib.BF16
    p.x = p.weight = p.dy = p.dx = p.dweight = 4096
    assert L.issm_b200_dwconv7_silu_bwd(C.byref(p), None) == 4                # no workspace
    need = L.issm_b200_dwconv_workspace_bytes(C.byref(p))
    assert need >= 2 * 290 * 8 * 4 and need % 256 == 0
    assert L.issm_b200_gather_rows(None, None, None, 1, 1, 1, 8, 8, 8, None, None) == 1
    assert L.issm_b200_gather_rows(4096, 4096, 4096, 1, 4, 4, 7, 28, 7, None, None) == 2   # odd row bytes
    with pytest.raises(RuntimeError):
        PointLiteConv(8, 8)(None, torch.randn(1, 10, 8))
    with pytest.raises(RuntimeError):
        reorder_points(torch.randn(1, 10, 8), torch.zeros(1, 10, dtype=torch.int64))
    with pytest.raises(ValueError):
        PointLiteConv(8, 16)


def test_parameter_generation_and_slice_entry_points_validate(built_lib):
    """issm_b200_glue_* and issm_b200_dt_sum: struct layout and the codes returned before any launch."""
    import torch
    from dest3d_b200 import _lib
    from dest3d_b200.adaptive_params import adaptive_dt_bc
    L = _lib.lib()
    assert L.issm_b200_sizeof_glue_params() == C.sizeof(_lib.IssmGlueParams)
    p = _lib.IssmGlueParams()
    assert L.issm_b200_glue_fwd(None, None) == 1
    p.batch, p.seqlen, p.nstates, p.nfeat, p.nheads, p.ngroups = 2, 10, 256, 5, 8, 1
    assert L.issm_b200_glue_fwd(C.byref(p), None) == 2                        # 5 features: not 4, 8 or 16
    p.nfeat, p.nheads = 16, 15
    assert L.issm_b200_glue_fwd(C.byref(p), None) == 2                        # more rows than a thread holds
    p.nheads, p.io_dtype = 8, _lib.BF16
    assert L.issm_b200_glue_fwd(C.byref(p), None) == 1                        # null pointers
    p.dist = p.weight = p.tok = p.dt = p.bc = p.ddist = p.dweight = p.dtok = 4096
    p.dist_sb, p.dist_sl, p.dist_sk = 10 * 256 * 16, 256 * 16, 16
    assert L.issm_b200_glue_bwd(C.byref(p), None) == 4                        # no workspace
    p.dist = 4098
    assert L.issm_b200_glue_fwd(C.byref(p), None) == 5                        # feature rows must be 16-byte aligned
    assert L.issm_b200_glue_workspace_bytes(C.byref(p)) % 256 == 0
    assert L.issm_b200_dt_sum(None, 0, 1, 1, 1, 1, 1, 1, 1, None, 0, 0.0, 1.0, 256, None, None) == 1
    assert L.issm_b200_dt_sum(4096, 0, 1, 0, 1, 1, 1, 1, 1, None, 0, 0.0, 1.0, 256, 4096, None) == 2
    assert L.issm_b200_dt_sum(4096, 7, 1, 8, 1, 1, 1, 1, 1, None, 0, 0.0, 1.0, 256, 4096, None) == 3
    with pytest.raises(RuntimeError):
        adaptive_dt_bc(torch.randn(1, 4, 8, 4), torch.randn(2, 4), torch.randn(2, 4), torch.randn(1, 4, 2), torch.randn(2),
                       torch.randn(1, 4, 1), torch.randn(1, 4, 1))


def test_strides_of_size_one_dimensions_do_not_select_the_slow_path(built_lib):
    """A (b, L, 1, N) sum of broadcast views reaches the library with group stride 1, and a batch of one with any batch
    stride: neither is ever used for addressing, so neither may fail the tensor-core path's alignment rules
    (models/dest_module.py:546-547 builds B and C exactly like that)."""
    from dest3d_b200 import _lib
    p = _params(batch=1, seqlen=384, nheads=8, headdim=36, dstate=256, ngroups=1, chunk_size=256, io_dtype=_lib.BF16, dt_dtype=_lib.F32,
                path=_lib.PATH_AUTO)
    p.x_sb, p.x_sl, p.x_sh = 384 * 288, 288, 36
    p.out_sb, p.out_sl, p.out_sh = 384 * 288, 288, 36
    p.dout_sb, p.dout_sl, p.dout_sh = 384 * 288, 288, 36
    p.dt_sb, p.dt_sl, p.dt_sh = 384 * 2048, 2048, 256
    p.B_sb, p.B_sl, p.B_sg = 384 * 256, 256, 256
    p.C_sb, p.C_sl, p.C_sg = 384 * 256, 256, 256
    assert built_lib.issm_b200_resolve_path_pass(C.byref(p), 0) == _lib.PATH_TENSOR
    p.B_sg = p.C_sg = 1                                                        # what torch reports for the size-one group axis
    p.x_sb = p.dt_sb = p.B_sb = 7                                              # and any value for a batch of one
    assert built_lib.issm_b200_resolve_path_pass(C.byref(p), 0) == _lib.PATH_TENSOR
    assert built_lib.issm_b200_resolve_path_pass(C.byref(p), 1) == _lib.PATH_TENSOR
    p.ngroups, p.nheads = 2, 8                                                 # with two groups the stride is real again
    p.B_sl = p.C_sl = 512
    assert built_lib.issm_b200_resolve_path_pass(C.byref(p), 0) == _lib.PATH_SIMT
