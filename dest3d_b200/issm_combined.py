"""ISSM chunked scan: the reference's Python interface on top of the B200 C ABI.

Mirrors `issm_triton/issm_combined.py:16-54` of the reference: `ISSM_chunk_scan_combined` has the
same positional/keyword arguments, return convention and gradient dtypes, so
`models/dest_module.py:600-611` can call it unchanged.  Two keyword-only extensions:
`reverse=True` scans from the last point to the first without flipped copies (what
models/dest_module.py:567-573 does with four torch.flip calls), and `path` selects the kernels
("auto", "simt", "tensor").

Two bindings reach the C ABI.  The default is the torch C++ extension (`torch.ops.issm_b200.fwd / bwd`,
csrc/issm_torch.cpp), which validates, allocates and fills the parameter struct in C++.  The ctypes binding of
`_lib.py` does the same from Python; it documents how any foreign-language host binds the library and is what
the tests use when they need to control every buffer of a call.  `BINDING` (or the environment variable
ISSM_B200_BINDING = "torch" | "ctypes") selects one; both fail loudly when the built library is missing.
"""
import ctypes as ct
import math
import os

import torch

from . import _ext, _lib

BINDING = os.environ.get("ISSM_B200_BINDING", "torch")
_PATHS = {"auto": _lib.PATH_AUTO, "simt": _lib.PATH_SIMT, "tensor": _lib.PATH_TENSOR}
_STATUS = {}


def _status_word(device):
    """One int32 per device that kernels OR error bits into (bit 0 (value 1): a bounded wait
    expired; bit 2 (value 4), informational: a 64-point block exceeded the decay range of the fast tensor-core
    kernel and its stream was redone by the windowed kernel)."""
    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    if key not in _STATUS:
        _STATUS[key] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", key))
    return _STATUS[key]


def device_status(device=None, reset=True):
    """Read (and by default clear) the device status word; synchronises the device."""
    w = _status_word(device if device is not None else torch.cuda.current_device())
    v = int(w.item())
    if reset and v:
        w.zero_()
    return v


def _empty(shape, dtype, device):
    """Every output and workspace buffer of this module is allocated here (one place for the tests to
    substitute an allocator that surrounds each buffer with guard bands)."""
    return torch.empty(tuple(shape), dtype=dtype, device=device)


def _row_major_last(t):
    """Kernels need a unit stride in the last dimension (the reference has the same rule,
    issm_combined.py:72-81)."""
    return t if t.stride(-1) == 1 else t.contiguous()


def _fill_common(x, dt, A, B, C, chunk_size, D, z, dt_bias, initial_states, dt_softplus, dt_limit,
                 reverse, path):
    """Validate like the reference (issm_combined.py:58-82) and build the parameter struct.
    Returns (params, keepalive list)."""
    if not x.is_cuda:
        raise RuntimeError("ISSM_chunk_scan_combined runs on CUDA tensors only; there is no CPU path")
    batch, seqlen, nheads, headdim = x.shape
    _, _, ngroups, dstate = B.shape
    assert nheads % ngroups == 0
    assert B.shape == (batch, seqlen, ngroups, dstate)
    assert dt.shape == (batch, seqlen, nheads, dstate)
    assert A.shape == (nheads, dstate)
    assert C.shape == B.shape
    if z is not None:
        assert z.shape == x.shape
    if D is not None:
        assert D.shape == (nheads, headdim) or D.shape == (nheads,)
    if initial_states is not None:
        assert initial_states.shape == (batch, nheads, headdim, dstate)
    io = x.dtype
    keep = []

    def act(t):
        t = _row_major_last(t if t.dtype == io else t.to(io))
        keep.append(t)
        return t

    def par(t):
        t = t.detach().to(torch.float32).contiguous()
        keep.append(t)
        return t

    xk, Bk, Ck = act(x), act(B), act(C)
    zk = act(z) if z is not None else None
    dtk = _row_major_last(dt if dt.dtype in (torch.float32, torch.bfloat16) else dt.float())
    keep.append(dtk)
    Ak = par(A)
    Dk = par(D) if D is not None else None
    if dt_bias is not None:
        bias = dt_bias if dt_bias.dim() == 2 else dt_bias[:, None].expand(nheads, dstate)
        assert bias.shape == (nheads, dstate)
        bk = par(bias)
    else:
        bk = None
    ik = None
    if initial_states is not None:
        ik = initial_states.to(io).contiguous()
        keep.append(ik)

    p = _lib.IssmParams()
    p.batch, p.seqlen, p.nheads, p.headdim, p.dstate, p.ngroups, p.chunk_size = batch, seqlen, nheads, headdim, dstate, ngroups, int(chunk_size)
    p.io_dtype, p.dt_dtype = _lib.dtype_code(io), _lib.dtype_code(dtk.dtype)
    p.path = _PATHS[path]
    p.has_D, p.D_has_hdim = int(D is not None), int(D is not None and D.dim() == 2)
    p.has_z, p.has_dt_bias, p.dt_softplus = int(z is not None), int(dt_bias is not None), int(bool(dt_softplus))
    p.has_init, p.reverse = int(initial_states is not None), int(bool(reverse))
    p.dt_min, p.dt_max = float(dt_limit[0]), float(min(dt_limit[1], 3.0e38))
    p.x, p.x_sb, p.x_sl, p.x_sh = xk.data_ptr(), xk.stride(0), xk.stride(1), xk.stride(2)
    p.dt, p.dt_sb, p.dt_sl, p.dt_sh = dtk.data_ptr(), dtk.stride(0), dtk.stride(1), dtk.stride(2)
    p.B, p.B_sb, p.B_sl, p.B_sg = Bk.data_ptr(), Bk.stride(0), Bk.stride(1), Bk.stride(2)
    p.C, p.C_sb, p.C_sl, p.C_sg = Ck.data_ptr(), Ck.stride(0), Ck.stride(1), Ck.stride(2)
    if zk is not None:
        p.z, p.z_sb, p.z_sl, p.z_sh = zk.data_ptr(), zk.stride(0), zk.stride(1), zk.stride(2)
    p.A, p.D, p.dt_bias, p.initial_states = Ak.data_ptr(), _lib.ptr(Dk), _lib.ptr(bk), _lib.ptr(ik)
    p.status = _status_word(x.device).data_ptr()
    return p, keep


class _StatusMirror:
    """Pinned host copy of one device's status word.  After every call an asynchronous 4-byte copy of the word
    is enqueued behind the call's kernels; the next call on that device (or `raise_on_device_error`) looks at the
    copy once it has landed.  An expired device-side wait therefore surfaces as a Python exception at the first
    call made after the failing kernels have finished and a copy enqueued behind them has landed (one copy is in flight
    at a time), without this module ever blocking on the device."""

    def __init__(self, device):
        self.host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.event = torch.cuda.Event()
        self.pending = False
        self.device = device

    def poll(self, what):
        if self.pending and self.event.query():
            self.pending = False
            v = int(self.host[0])
            if v & 1:
                self.host.zero_()
                _status_word(self.device).zero_()
                raise RuntimeError(f"{what}: a bounded device-side wait expired in an earlier ISSM call on {self.device} "
                                   f"(status {v}); the results of that call are invalid")

    def refresh(self):
        if torch.cuda.is_current_stream_capturing():
            return
        self.host.copy_(_status_word(self.device), non_blocking=True)
        self.event.record()
        self.pending = True


_MIRROR = {}


def _check_status(device, what):
    """Surfaces device status bit 0 (a bounded wait expired).  Default: asynchronously, see _StatusMirror.  With
    ISSM_B200_CHECK_STATUS=1 every call synchronises and raises at once (debug aid).  Bit 2 of the word is
    informational: some 64-point block exceeded the range of the single-reference factorisation and its stream
    was redone by the windowed kernels."""
    if os.environ.get("ISSM_B200_CHECK_STATUS") == "1":
        raise_on_device_error(device, what)
        return
    dev = torch.device(device)
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    m = _MIRROR.get(key)
    if m is None:
        m = _MIRROR[key] = _StatusMirror(torch.device("cuda", key))
    with torch.cuda.device(key):
        if torch.cuda.is_current_stream_capturing():     # inside a CUDA-graph capture: neither query nor copy
            return
        m.poll(what)
        if not m.pending:                                # one copy in flight at a time: a step of several calls enqueues one
            m.refresh()


def raise_on_device_error(device=None, what="ISSM"):
    """Synchronise the device and raise if any ISSM call since the last check recorded an expired wait (status
    bit 0); the word is cleared.  Call it at a point where the training loop synchronises anyway."""
    v = device_status(device)
    if v & 1:
        raise RuntimeError(f"{what}: a bounded device-side wait expired (status {v}); results are invalid")


def _workspace(p, pass_, device, keep):
    need = _lib.lib().issm_b200_workspace_bytes(ct.byref(p), pass_)
    ws = _empty((max(int(need), 256),), torch.uint8, device)
    keep.append(ws)
    p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()


def issm_fwd(x, dt, A, B, C, chunk_size, D=None, z=None, dt_bias=None, initial_states=None,
             dt_softplus=False, dt_limit=(0.0, float("inf")), reverse=False, path="auto",
             want_final=True, save_states=False):
    """Forward only (no autograd).  Returns (out, out_x or None, final_states or None), plus the
    saved block-entry states (or None) when `save_states` is set; counterpart of
    `_issm_chunk_scan_combined_fwd` (issm_combined.py:57-92)."""
    if BINDING == "torch":
        out, out_x, final, saved = _ext.ops().fwd(
            x, dt, A, B, C, int(chunk_size), D, z, dt_bias, initial_states, bool(dt_softplus), float(dt_limit[0]),
            float(dt_limit[1]), bool(reverse), _PATHS[path], bool(want_final), bool(save_states), _status_word(x.device))
        _check_status(x.device, "issm_b200_fwd")
        out_x, final, saved = _ext.opt(out_x), _ext.opt(final), _ext.opt(saved)
        return (out, out_x, final, saved) if save_states else (out, out_x, final)
    p, keep = _fill_common(x, dt, A, B, C, chunk_size, D, z, dt_bias, initial_states, dt_softplus,
                           dt_limit, reverse, path)
    saved = None
    if save_states and _lib.lib().issm_b200_resolve_path_pass(ct.byref(p), 1) == _lib.PATH_TENSOR:
        # the tensor-core backward reads the state entering every 64-point block instead of recomputing it
        saved = _empty((x.shape[0], x.shape[2], (x.shape[1] + 63) // 64 + 1, B.shape[-1], 48), torch.bfloat16, x.device)
        p.saved_states = saved.data_ptr()
    out = _empty(x.shape, x.dtype, x.device)
    out_x = _empty(x.shape, x.dtype, x.device) if z is not None else None
    final = _empty((x.shape[0], x.shape[2], x.shape[3], B.shape[-1]), torch.float32, x.device) if want_final else None
    p.out, p.out_sb, p.out_sl, p.out_sh = out.data_ptr(), out.stride(0), out.stride(1), out.stride(2)
    p.out_x, p.final_states, p.want_final = _lib.ptr(out_x), _lib.ptr(final), int(want_final)
    _workspace(p, 0, x.device, keep)
    with torch.cuda.device(x.device):
        rc = _lib.lib().issm_b200_fwd(ct.byref(p), _lib.stream_ptr(x.device))
    if rc:
        raise _lib.IssmError(rc, "issm_b200_fwd")
    _check_status(x.device, "issm_b200_fwd")
    return (out, out_x, final, saved) if save_states else (out, out_x, final)


def issm_bwd(dout, x, dt, A, B, C, out_x, chunk_size, D=None, z=None, dt_bias=None,
             initial_states=None, dfinal_states=None, dt_softplus=False,
             dt_limit=(0.0, float("inf")), reverse=False, path="auto", saved_states=None):
    """Backward; counterpart of `_issm_chunk_scan_combined_bwd` (issm_combined.py:95-179).
    `out_x` is the pre-gate output saved by the forward (only read when z is given).
    Returns (dx, ddt, dA, dB, dC, dD, dz, ddt_bias, dinitial_states) with the reference's dtypes;
    dA / dD / ddt_bias are float32 here and cast by the caller."""
    if BINDING == "torch":
        res = _ext.ops().bwd(dout, x, dt, A, B, C, out_x, int(chunk_size), D, z, dt_bias, initial_states, dfinal_states,
                             bool(dt_softplus), float(dt_limit[0]), float(dt_limit[1]), bool(reverse), _PATHS[path],
                             saved_states, _status_word(x.device))
        _check_status(x.device, "issm_b200_bwd")
        dx, ddt, dA, dB, dC, dD, dz, dbias, dinit = res
        return dx, ddt, dA, dB, dC, _ext.opt(dD), _ext.opt(dz), _ext.opt(dbias), _ext.opt(dinit)
    p, keep = _fill_common(x, dt, A, B, C, chunk_size, D, z, dt_bias, initial_states, dt_softplus,
                           dt_limit, reverse, path)
    dev = x.device
    io = x.dtype
    doutk = _row_major_last(dout if dout.dtype == io else dout.to(io))
    keep.append(doutk)
    H, N = A.shape
    dx = _empty(x.shape, io, dev)
    ddt = _empty(dt.shape, torch.float32 if p.dt_dtype == _lib.F32 else torch.bfloat16, dev)
    dB = _empty(B.shape, io, dev)
    dC = _empty(C.shape, io, dev)
    dz = _empty(x.shape, io, dev) if z is not None else None
    dA = _empty((H, N), torch.float32, dev)
    dbias = _empty((H, N), torch.float32, dev) if dt_bias is not None else None
    dD = _empty(D.shape, torch.float32, dev) if D is not None else None
    dinit = _empty(initial_states.shape, io, dev) if initial_states is not None else None
    if z is not None:
        # out_x was allocated contiguous by the forward
        assert out_x is not None and out_x.is_contiguous()
        p.out_x = out_x.data_ptr()
        p.out_sb, p.out_sl, p.out_sh = out_x.stride(0), out_x.stride(1), out_x.stride(2)
    p.dout, p.dout_sb, p.dout_sl, p.dout_sh = doutk.data_ptr(), doutk.stride(0), doutk.stride(1), doutk.stride(2)
    if dfinal_states is not None:
        dfin = dfinal_states.to(torch.float32).contiguous()
        keep.append(dfin)
        p.has_dfinal, p.dfinal_states = 1, dfin.data_ptr()
    p.dx, p.ddt, p.dB, p.dC, p.dz = dx.data_ptr(), ddt.data_ptr(), dB.data_ptr(), dC.data_ptr(), _lib.ptr(dz)
    p.dA, p.ddt_bias, p.dD, p.dinitial_states = dA.data_ptr(), _lib.ptr(dbias), _lib.ptr(dD), _lib.ptr(dinit)
    p.saved_states = _lib.ptr(saved_states)
    _workspace(p, 1, dev, keep)
    with torch.cuda.device(dev):
        rc = _lib.lib().issm_b200_bwd(ct.byref(p), _lib.stream_ptr(dev))
    if rc:
        raise _lib.IssmError(rc, "issm_b200_bwd")
    _check_status(dev, "issm_b200_bwd")
    return dx, ddt, dA, dB, dC, dD, dz, dbias, dinit


class ISSMChunkScanCombinedFn(torch.autograd.Function):
    """autograd entry, same saved-tensor and return conventions as the reference
    (issm_combined.py:37-54); two trailing extras (reverse, path) receive no gradient."""

    @staticmethod
    def forward(ctx, x, dt, A, B, C, chunk_size, D=None, z=None, dt_bias=None, initial_states=None,
                seq_idx=None, dt_softplus=False, dt_limit=(0.0, float("inf")), return_final_states=False,
                reverse=False, path="auto"):
        assert seq_idx is None, "ISSM_chunk_scan_combined splits packed batches before it reaches the autograd function"
        need_grad = any(ctx.needs_input_grad)
        res = issm_fwd(x, dt, A, B, C, chunk_size, D, z, dt_bias, initial_states, dt_softplus, dt_limit,
                       reverse, path, want_final=return_final_states, save_states=need_grad)
        out, out_x, final = res[:3]
        saved = res[3] if need_grad else None
        ctx.save_for_backward(out_x, x, dt, A, B, C, D, z, dt_bias, initial_states, saved)
        ctx.opts = (chunk_size, dt_softplus, dt_limit, return_final_states, reverse, path)
        return out if not return_final_states else (out, final)

    @staticmethod
    def backward(ctx, dout, *args):
        out_x, x, dt, A, B, C, D, z, dt_bias, initial_states, saved = ctx.saved_tensors
        chunk_size, dt_softplus, dt_limit, return_final_states, reverse, path = ctx.opts
        dfinal = args[0] if return_final_states and len(args) and args[0] is not None else None
        dx, ddt, dA, dB, dC, dD, dz, dbias, dinit = issm_bwd(
            dout, x, dt, A, B, C, out_x, chunk_size, D, z, dt_bias, initial_states, dfinal,
            dt_softplus, dt_limit, reverse, path, saved_states=saved)
        ddt = ddt if ddt.dtype == dt.dtype else ddt.to(dt.dtype)
        dA = dA.to(A.dtype)
        dB = dB if dB.dtype == B.dtype else dB.to(B.dtype)
        dC = dC if dC.dtype == C.dtype else dC.to(C.dtype)
        if dD is not None:
            dD = dD.to(D.dtype)
        if dz is not None and dz.dtype != z.dtype:
            dz = dz.to(z.dtype)
        if dbias is not None:
            dbias = (dbias if dt_bias.dim() == 2 else dbias.sum(dim=1)).to(dt_bias.dtype)
        if dinit is not None and dinit.dtype != initial_states.dtype:
            dinit = dinit.to(initial_states.dtype)
        return dx, ddt, dA, dB, dC, None, dD, dz, dbias, dinit, None, None, None, None, None, None


def ISSM_chunk_scan_combined(x, dt, A, B, C, chunk_size, D=None, z=None, dt_bias=None, initial_states=None,
                             seq_idx=None, dt_softplus=False, dt_limit=(0.0, float("inf")),
                             return_final_states=False, *, reverse=False, path="auto", slices=1):
    """
    Argument:
        x: (batch, seqlen, nheads, headdim)
        dt: (batch, seqlen, nheads, dstate)
        A: (nheads, dstate)
        B: (batch, seqlen, ngroups, dstate)
        C: (batch, seqlen, ngroups, dstate)
        chunk_size: int (<= 256)
        D: (nheads, headdim) or (nheads,)
        z: (batch, seqlen, nheads, headdim)
        dt_bias: (nheads, dstate) or (nheads,)
        initial_states: (batch, nheads, headdim, dstate)
        seq_idx: (batch, seqlen) or None; sequences packed along seqlen, no state crosses a change of seq_idx
        dt_softplus: Whether to apply softplus to dt
        slices (extension): cut every sequence into this many slices that run as extra batch entries (two passes; for
            few, long sequences - one CTA serves one (sample, head) stream); "auto" picks the count from the sizes
    Return:
        out: (batch, seqlen, nheads, headdim), or (out, final_states (batch, nheads, headdim, dstate) fp32)
    """
    if slices != 1 and seq_idx is None:
        from .seqpar import issm_scan_chunk_parallel
        return issm_scan_chunk_parallel(x, dt, A, B, C, chunk_size, D=D, z=z, dt_bias=dt_bias, initial_states=initial_states,
                                        dt_softplus=dt_softplus, dt_limit=dt_limit, return_final_states=return_final_states,
                                        reverse=reverse, path=path, slices=None if slices == "auto" else int(slices))
    if seq_idx is not None:
        return _scan_packed(x, dt, A, B, C, chunk_size, D, z, dt_bias, initial_states, seq_idx, dt_softplus, dt_limit,
                            return_final_states, reverse, path)
    return ISSMChunkScanCombinedFn.apply(x, dt, A, B, C, chunk_size, D, z, dt_bias, initial_states, None,
                                         dt_softplus, dt_limit, return_final_states, reverse, path)


def _scan_packed(x, dt, A, B, C, chunk_size, D, z, dt_bias, initial_states, seq_idx, dt_softplus, dt_limit,
                 return_final_states, reverse, path):
    """seq_idx (batch, seqlen): several sequences packed along seqlen; no state flows from one to the next.

    The reference threads seq_idx through every kernel: the state is multiplied by zero wherever seq_idx changes
    (issm_triton/issm_state_passing.py:92-99), rows only see earlier rows of their own sequence
    (issm_triton/issm_cabt_bmm.py:14) and the incoming state only reaches rows whose seq_idx equals that of the
    row before (issm_triton/issm_chunk_scan.py:122-131), where the row "before the first" counts as sequence 0 -
    so initial_states only enter when the first sequence has index 0.  For the usual packed layout (each sequence
    one contiguous run of seq_idx) that is exactly one independent scan per run, which is how it is done here: the
    runs are found on the host (one device-to-host copy of seq_idx) and every run is one call of the kernels on a
    view of the inputs; autograd stitches the gradients.  final_states are those of the last run in scan order."""
    batch, seqlen = x.shape[0], x.shape[1]
    assert seq_idx.shape == (batch, seqlen)
    idx = seq_idx.detach().to("cpu")
    outs, finals = [], []
    for b in range(batch):
        row = idx[b]
        change = (torch.nonzero(row[1:] != row[:-1]).flatten() + 1).tolist()
        bounds = [0] + change + [seqlen]
        runs = list(zip(bounds[:-1], bounds[1:]))
        first = runs[-1] if reverse else runs[0]           # the run the scan enters first
        ys, fin = [], None
        for (s, e) in (reversed(runs) if reverse else runs):
            init = None
            if initial_states is not None and (s, e) == first and int(row[e - 1 if reverse else s]) == 0:
                init = initial_states[b:b + 1]
            sl = lambda t: None if t is None else t[b:b + 1, s:e]
            y, fin = ISSMChunkScanCombinedFn.apply(sl(x), sl(dt), A, sl(B), sl(C), chunk_size, D, sl(z), dt_bias, init, None,
                                                   dt_softplus, dt_limit, True, reverse, path)
            ys.append(y)
        outs.append(torch.cat(ys[::-1] if reverse else ys, dim=1))
        finals.append(fin)
    out = torch.cat(outs, dim=0)
    return (out, torch.cat(finals, dim=0)) if return_final_states else out


def issm_bidirectional_scan(x, x_back, dt, A, B, C, B_back, C_back, chunk_size, D=None, z=None, dt_bias=None,
                            initial_states=None, dt_softplus=False, dt_limit=(0.0, float("inf")),
                            out_scale=0.5, path="auto"):
    """Forward scan of (x, B, C) plus reversed scan of (x_back, B_back, C_back) over the SAME dt, A, D,
    initial states, combined as out_scale * (fwd + bwd): the bidirectional block of
    models/dest_module.py:565-575 (which averages, out_scale = 0.5) without the flipped copies.
    All `_back` tensors are in natural point order.  Returns (out, final_states)."""
    yf, sf = ISSM_chunk_scan_combined(x, dt, A, B, C, chunk_size, D, z, dt_bias, initial_states, None,
                                      dt_softplus, dt_limit, True, reverse=False, path=path)
    yb, sb = ISSM_chunk_scan_combined(x_back, dt, A, B_back, C_back, chunk_size, D, z, dt_bias, initial_states,
                                      None, dt_softplus, dt_limit, True, reverse=True, path=path)
    return (yf + yb) * out_scale, (sf + sb) * out_scale
