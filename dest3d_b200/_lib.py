"""ctypes binding of libissm_b200.so (the C ABI declared in include/issm_b200.h).

The library is the product: importing this module without it raises, there is no fallback.
"""
import ctypes as C
import os

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_PKG, "libissm_b200.so")

F32, BF16 = 0, 1
PATH_AUTO, PATH_SIMT, PATH_TENSOR = 0, 1, 2
_DTYPES = {torch.float32: F32, torch.bfloat16: BF16}

i32, i64, f32, vp = C.c_int32, C.c_int64, C.c_float, C.c_void_p


class IssmParams(C.Structure):
    """Mirror of `issm_params` (include/issm_b200.h); field order and types must match."""
    _fields_ = (
        [(n, i32) for n in ("batch", "seqlen", "nheads", "headdim", "dstate", "ngroups", "chunk_size",
                            "io_dtype", "dt_dtype", "path",
                            "has_D", "D_has_hdim", "has_z", "has_dt_bias", "dt_softplus",
                            "has_init", "has_dfinal", "reverse", "want_final")]
        + [("dt_min", f32), ("dt_max", f32)]
        + [("x", vp), ("x_sb", i64), ("x_sl", i64), ("x_sh", i64)]
        + [("dt", vp), ("dt_sb", i64), ("dt_sl", i64), ("dt_sh", i64)]
        + [("B", vp), ("B_sb", i64), ("B_sl", i64), ("B_sg", i64)]
        + [("C", vp), ("C_sb", i64), ("C_sl", i64), ("C_sg", i64)]
        + [("z", vp), ("z_sb", i64), ("z_sl", i64), ("z_sh", i64)]
        + [("A", vp), ("D", vp), ("dt_bias", vp), ("initial_states", vp)]
        + [("out", vp), ("out_sb", i64), ("out_sl", i64), ("out_sh", i64), ("out_x", vp), ("final_states", vp)]
        + [("dout", vp), ("dout_sb", i64), ("dout_sl", i64), ("dout_sh", i64), ("dfinal_states", vp)]
        + [(n, vp) for n in ("dx", "ddt", "dB", "dC", "dz", "dA", "ddt_bias", "dD", "dinitial_states")]
        + [("workspace", vp), ("workspace_bytes", C.c_size_t), ("status", vp), ("saved_states", vp)]
    )


class IssmNormParams(C.Structure):
    """Mirror of `issm_norm_params`."""
    _fields_ = (
        [(n, i32) for n in ("rows", "hidden", "group_size", "io_dtype", "is_rms", "norm_before_gate", "has_z", "has_bias")]
        + [("eps", f32)]
        + [("x", vp), ("x_sr", i64), ("z", vp), ("z_sr", i64), ("weight", vp), ("bias", vp),
           ("y", vp), ("y_sr", i64), ("rstd", vp), ("mean", vp),
           ("dy", vp), ("dy_sr", i64), ("dx", vp), ("dz", vp), ("dweight", vp), ("dbias", vp),
           ("workspace", vp), ("workspace_bytes", C.c_size_t)]
    )


class IssmConvParams(C.Structure):
    """Mirror of `issm_conv_params`."""
    _fields_ = (
        [(n, i32) for n in ("batch", "seqlen", "channels", "io_dtype")]
        + [("x", vp), ("x_sb", i64), ("x_sl", i64), ("weight", vp), ("bias", vp), ("y", vp),
           ("dy", vp), ("dy_sb", i64), ("dy_sl", i64), ("dx", vp), ("dweight", vp), ("dbias", vp),
           ("workspace", vp), ("workspace_bytes", C.c_size_t)]
    )


class IssmGlueParams(C.Structure):
    """Mirror of `issm_glue_params`."""
    _fields_ = (
        [(n, i32) for n in ("batch", "seqlen", "nstates", "nfeat", "nheads", "ngroups", "has_back", "io_dtype", "dist_dtype")]
        + [("dist", vp), ("dist_sb", i64), ("dist_sl", i64), ("dist_sk", i64), ("weight", vp), ("tok", vp), ("mask", vp),
           ("dt", vp), ("bc", vp), ("ddt", vp), ("dbc", vp), ("ddist", vp), ("dweight", vp), ("dtok", vp),
           ("workspace", vp), ("workspace_bytes", C.c_size_t)]
    )


class IssmError(RuntimeError):
    def __init__(self, code, what):
        self.code = code
        super().__init__(f"{what}: error {code}: {lib().issm_b200_strerror(code).decode()}")


_lib = None


def lib():
    """Load the shared library once; raise loudly when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_LIB_PATH):
        raise RuntimeError(
            f"{_LIB_PATH} is missing: the CUDA library has not been built. Run `python -m dest3d_b200.build` "
            "(needs nvcc); there is no CPU or PyTorch fallback.")
    L = C.CDLL(_LIB_PATH)
    L.issm_b200_version.restype = C.c_int
    L.issm_b200_strerror.restype = C.c_char_p
    L.issm_b200_strerror.argtypes = [C.c_int]
    for name in ("issm_b200_sizeof_params", "issm_b200_sizeof_norm_params", "issm_b200_sizeof_conv_params"):
        getattr(L, name).restype = C.c_size_t
    L.issm_b200_workspace_bytes.restype = C.c_size_t
    L.issm_b200_workspace_bytes.argtypes = [C.POINTER(IssmParams), C.c_int]
    L.issm_b200_resolve_path.restype = C.c_int
    L.issm_b200_resolve_path.argtypes = [C.POINTER(IssmParams)]
    L.issm_b200_resolve_path_pass.restype = C.c_int
    L.issm_b200_resolve_path_pass.argtypes = [C.POINTER(IssmParams), C.c_int]
    for name in ("issm_b200_fwd", "issm_b200_bwd"):
        getattr(L, name).restype = C.c_int
        getattr(L, name).argtypes = [C.POINTER(IssmParams), vp]
    L.issm_b200_norm_workspace_bytes.restype = C.c_size_t
    L.issm_b200_norm_workspace_bytes.argtypes = [C.POINTER(IssmNormParams), C.c_int]
    for name in ("issm_b200_norm_fwd", "issm_b200_norm_bwd"):
        getattr(L, name).restype = C.c_int
        getattr(L, name).argtypes = [C.POINTER(IssmNormParams), vp]
    L.issm_b200_dwconv_workspace_bytes.restype = C.c_size_t
    L.issm_b200_dwconv_workspace_bytes.argtypes = [C.POINTER(IssmConvParams)]
    for name in ("issm_b200_dwconv7_silu_fwd", "issm_b200_dwconv7_silu_bwd"):
        getattr(L, name).restype = C.c_int
        getattr(L, name).argtypes = [C.POINTER(IssmConvParams), vp]
    L.issm_b200_gather_rows.restype = C.c_int
    L.issm_b200_gather_rows.argtypes = [vp, vp, vp, i32, i32, i32, i64, i64, i64, vp, vp]
    L.issm_b200_sizeof_glue_params.restype = C.c_size_t
    L.issm_b200_glue_workspace_bytes.restype = C.c_size_t
    L.issm_b200_glue_workspace_bytes.argtypes = [C.POINTER(IssmGlueParams)]
    for name in ("issm_b200_glue_fwd", "issm_b200_glue_bwd"):
        getattr(L, name).restype = C.c_int
        getattr(L, name).argtypes = [C.POINTER(IssmGlueParams), vp]
    if L.issm_b200_sizeof_glue_params() != C.sizeof(IssmGlueParams):
        raise RuntimeError("libissm_b200.so and dest3d_b200/_lib.py disagree on issm_glue_params; rebuild")
    L.issm_b200_dt_sum.restype = C.c_int
    L.issm_b200_dt_sum.argtypes = [vp, i32, i32, i32, i32, i32, i64, i64, i64, vp, i32, f32, f32, i32, vp, vp]
    L.issm_b200_launch_count.restype = C.c_uint64
    if L.issm_b200_sizeof_conv_params() != C.sizeof(IssmConvParams):
        raise RuntimeError("libissm_b200.so and dest3d_b200/_lib.py disagree on issm_conv_params; rebuild")
    if L.issm_b200_sizeof_params() != C.sizeof(IssmParams) or L.issm_b200_sizeof_norm_params() != C.sizeof(IssmNormParams):
        raise RuntimeError("libissm_b200.so and dest3d_b200/_lib.py disagree on the parameter struct layout; rebuild")
    _lib = L
    return L


def dtype_code(t):
    try:
        return _DTYPES[t]
    except KeyError:
        raise TypeError(f"unsupported dtype {t}: the ISSM kernels take float32 or bfloat16") from None


def ptr(t):
    return None if t is None else t.data_ptr()


def stream_ptr(device):
    return torch.cuda.current_stream(device).cuda_stream


def launch_count():
    return int(lib().issm_b200_launch_count())
