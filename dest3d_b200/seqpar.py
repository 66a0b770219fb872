"""Sequence-parallel scan: ONE long sequence split along the point axis over several GPUs.

The state recurrence is linear in the state, so a rank's slice acts on the state entering it as
    S_out = Dec * S_in + F,      Dec[h, n] = exp(A[h, n] * sum_l dt[l, h, n]),   F = the slice's final state from S_in = 0,
which is how the reference chains its chunks (issm_triton/issm_state_passing.py:92-107, one (decay, state) pair per
chunk).  Here a rank plays the role of a chunk:

  forward   pass 1: every slice is scanned from a zero state -> F; Dec from the sums of the transformed dt;
            ONE all-gather of the (F, Dec) pairs (none on a single GPU); one sweep over the pairs in scan order gives
            the state entering every slice (the caller's initial state is folded into the first pair);
            pass 2: every slice again from the state entering it -> the output rows.
  backward  the same with the adjoint recurrence dS_in = Dec * dS_out + G, G = dS_in for dS_out = 0:
            pass 1 -> G; ONE all-gather of G (and of the gradient of the final state, taken from the last position);
            one sweep from the end -> dS_out of every slice; pass 2 with that dS_out -> all gradients.

A slice is a contiguous run of points.  On ONE GPU the slices of a sequence are folded into the batch axis, so that a
single long scene (batch 1, 8 heads: 8 of 148 SMs busy, one CTA per (sample, head) stream) runs b * R * H streams at
once; the reference pays nothing comparable because each of its chunks is its own program
(issm_triton/issm_chunk_state.py:234-356).  Over several GPUs every rank holds a contiguous part of the sequence,
cuts it into its own slices the same way, and the pairs of all ranks form one chain.  Every slice is scanned twice in
each direction of differentiation, so the gain is (streams that run at once) / 2.  Parameter gradients (dA, dD,
ddt_bias) of a rank are partial sums, to be all-reduced like in the data-parallel mode (`dist.PackedParamGrads`).
A reversed scan visits the slices, and the ranks, in descending order.  Carried states cross a slice boundary in the
input dtype (bf16 inputs: rounded to bf16 there, like the initial_states of any call)."""
import torch
import torch.distributed as dist

from . import issm_combined


def _wide(t):
    """Carried states are float32 (float64 inputs, which only the CPU checker produces, stay float64)."""
    return t if t.dtype == torch.float64 else t.float()


class Options:
    def __init__(self, chunk_size, dt_softplus=False, dt_limit=(0.0, float("inf")), reverse=False, path="auto"):
        self.chunk_size, self.dt_softplus, self.dt_limit, self.reverse, self.path = chunk_size, dt_softplus, dt_limit, reverse, path

    def kw(self):
        return dict(dt_softplus=self.dt_softplus, dt_limit=self.dt_limit, reverse=self.reverse, path=self.path)


def _slice_decay_cuda(dt, A, dt_bias, o):
    """exp(A * sum over the slice of the transformed dt), (b, H, 1, N) float32: the factor the slice applies to the
    state entering it.  The sums come from the library's `issm_b200_dt_sum` (one read of dt, fixed summation order)."""
    import ctypes as ct
    from . import _lib
    if not dt.is_cuda:
        raise RuntimeError("dest3d_b200.seqpar runs on CUDA tensors only")
    if dt.stride(3) != 1:
        dt = dt.contiguous()
    b, L, H, N = dt.shape
    bias = None
    if dt_bias is not None:
        bias = (dt_bias if dt_bias.dim() == 2 else dt_bias[:, None].expand(H, N)).float().contiguous()
    rows = 256
    part = torch.empty(((L + rows - 1) // rows, b, H, N), dtype=torch.float32, device=dt.device)
    with torch.cuda.device(dt.device):
        rc = _lib.lib().issm_b200_dt_sum(dt.data_ptr(), _lib.dtype_code(dt.dtype), b, L, H, N, dt.stride(0), dt.stride(1), dt.stride(2),
                                         _lib.ptr(bias), int(bool(o.dt_softplus)), float(o.dt_limit[0]), float(min(o.dt_limit[1], 3.0e38)),
                                         rows, part.data_ptr(), _lib.stream_ptr(dt.device))
    if rc:
        raise _lib.IssmError(rc, "issm_b200_dt_sum")
    return torch.exp(A.float() * part.sum(dim=0)).unsqueeze(2)


class KernelBackend:
    """The library's CUDA kernels (no autograd inside)."""
    fwd = staticmethod(issm_combined.issm_fwd)
    bwd = staticmethod(issm_combined.issm_bwd)
    decay = staticmethod(_slice_decay_cuda)


def states_entering(pairs, like):
    """From the (F, Dec) pairs of all positions, in scan order: ([state entering position 0 .. n - 1], final state);
    position 0 enters with zero (a caller's initial state is folded into its F beforehand)."""
    s, out = torch.zeros_like(like), []
    for f, dec in pairs:
        out.append(s)
        s = torch.addcmul(f, dec, s)
    return out, s


def grads_leaving(gpairs, dfinal, like):
    """From the (G, Dec) pairs of all positions and the gradient of the final state: the gradient of the state LEAVING
    every position, in one sweep from the end."""
    t = torch.zeros_like(like) if dfinal is None else _wide(dfinal)
    out = [None] * len(gpairs)
    for pos in range(len(gpairs) - 1, -1, -1):
        out[pos] = t
        g, dec = gpairs[pos]
        t = torch.addcmul(g, dec, t)
    return out


def forward_summary(be, o, x, dt, A, B, C, D, z, dt_bias):
    """Forward pass 1: the slices' final states from a zero entering state (the gate z does not touch the state, so
    it is left out), and their decays.  Returns (F, Dec)."""
    with torch.no_grad():
        res = be.fwd(x, dt, A, B, C, o.chunk_size, D, None, dt_bias, None, want_final=True, **o.kw())
        return _wide(res[2]), be.decay(dt, A, dt_bias, o)


def forward_final(be, o, x, dt, A, B, C, D, z, dt_bias, s_in):
    """Forward pass 2: the slices from the states entering them.  Returns (out, out_x, None, saved block states)."""
    with torch.no_grad():
        return be.fwd(x, dt, A, B, C, o.chunk_size, D, z, dt_bias, s_in, want_final=False, save_states=True, **o.kw())


def backward_summary(be, o, dout, x, dt, A, B, C, D, z, dt_bias, s_in, out_x, saved):
    """Backward pass 1: G = gradient of the entering state when nothing arrives from the later slices."""
    with torch.no_grad():
        return be.bwd(dout, x, dt, A, B, C, out_x, o.chunk_size, D, z, dt_bias, s_in, None, saved_states=saved, **o.kw())[8]


def backward_final(be, o, dout, x, dt, A, B, C, D, z, dt_bias, s_in, out_x, saved, ds_out):
    """Backward pass 2 with the gradient of the leaving state.  Returns issm_bwd's tuple."""
    with torch.no_grad():
        return be.bwd(dout, x, dt, A, B, C, out_x, o.chunk_size, D, z, dt_bias, s_in, ds_out, saved_states=saved, **o.kw())




def pick_slices(batch, nheads, seqlen, sms=148, min_points=512, ranks=1):
    """Slices per (local) sequence so that batch * slices * nheads streams fill the SMs, each slice keeping at least
    `min_points` points; 1 when a quarter of the SMs is busy anyway (two passes would cost more than they gain)."""
    want = -(-sms // max(1, batch * nheads))
    if want < 4 and ranks == 1:
        return 1
    return max(1, min(want, seqlen // min_points))


def _layout(L, R):
    """(slice length, number of equal slices, tail points).  Prefers a slice count in (R / 2, R] that divides L."""
    for r in range(R, max(1, R // 2), -1):
        if L % r == 0:
            return L // r, r, 0
    lr = -(-L // R)
    return lr, L // lr, L % lr


class _Folded:
    """Point-axis tensors of b sequences regrouped as [b * Rf equal slices folded into the batch axis] (+ [tail])."""

    def __init__(self, L, R):
        self.L = L
        self.lr, self.rf, self.tail = _layout(L, R)
        self.n = self.rf + (1 if self.tail else 0)          # slices per sequence, in memory order
        self.groups = 2 if self.tail else 1

    def split(self, t):
        if t is None:
            return [None] * self.groups
        b = t.shape[0]
        main = t[:, :self.rf * self.lr].reshape(b * self.rf, self.lr, *t.shape[2:])
        return [main, t[:, self.rf * self.lr:]] if self.tail else [main]

    def merge(self, parts, b):
        main = parts[0].reshape(b, self.rf * self.lr, *parts[0].shape[2:])
        return torch.cat([main, parts[1]], dim=1) if self.tail else main

    def per_slice(self, parts, b):
        """List over the slices (memory order) of per-sequence tensors (b, ...), from per-group results."""
        main = parts[0].reshape(b, self.rf, *parts[0].shape[1:])
        out = [main[:, i] for i in range(self.rf)]
        return out + [parts[1]] if self.tail else out

    def per_group(self, slices):
        """Inverse of per_slice."""
        main = torch.stack(slices[:self.rf], dim=1)
        main = main.reshape(main.shape[0] * self.rf, *main.shape[2:])
        return [main, slices[self.rf]] if self.tail else [main]


class Solo:
    """The chain of a single process: no collective."""
    world, pos = 1, 0

    def gather(self, flat):
        return [flat]


class RankChain:
    """Scan position of this rank among the ranks of a torch.distributed group (ascending ranks for a forward scan,
    descending for a reversed one) and the one collective the mode uses."""

    def __init__(self, group=None, reverse=False):
        self.group = group
        self.world = dist.get_world_size(group)
        rank = dist.get_rank(group)
        self.pos = self.world - 1 - rank if reverse else rank
        self.reverse = reverse

    def gather(self, flat):
        """All-gather one flat buffer; returns the ranks' buffers in scan order."""
        bufs = [torch.empty_like(flat) for _ in range(self.world)]
        dist.all_gather(bufs, flat, group=self.group)
        return bufs[::-1] if self.reverse else bufs


def _exchange(chain, mine, slots, like):
    """`mine`: this rank's list of (a, dec) pairs in scan order, at most `slots` of them.  Pads the list with identity
    pairs (a = 0, dec = 1: they leave a chain unchanged) to `slots`, all-gathers, and returns the pairs of ALL ranks in
    scan order plus the index of this rank's first pair."""
    ones = torch.ones_like(mine[0][1])
    padded = list(mine) + [(like, ones)] * (slots - len(mine))
    flat = torch.cat([torch.cat([a.reshape(-1), d.reshape(-1)]) for a, d in padded])
    na, nd = like.numel(), ones.numel()
    pairs = []
    for buf in chain.gather(flat):
        for i in range(slots):
            o = i * (na + nd)
            pairs.append((buf[o:o + na].view(like.shape), buf[o + na:o + na + nd].view(ones.shape)))
    return pairs, chain.pos * slots


class SlicedScanFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, chain, be, o, R, x, dt, A, B, C, D, z, dt_bias, initial_states):
        b, L, H, P = x.shape
        fo = _Folded(L, R)
        like = torch.zeros((b, H, P, A.shape[1]), dtype=_wide(x).dtype, device=x.device)
        xs, dts, Bs, Cs, zs = (fo.split(t) for t in (x, dt, B, C, z))
        groups = range(fo.groups)
        summ = [forward_summary(be, o, xs[g], dts[g], A, Bs[g], Cs[g], D, None, dt_bias) for g in groups]
        f, dec = fo.per_slice([s[0] for s in summ], b), fo.per_slice([s[1] for s in summ], b)
        order = list(range(fo.n))[::-1] if o.reverse else list(range(fo.n))      # local slice at every local scan position
        mine = [(f[i], dec[i]) for i in order]
        first = chain.pos == 0
        if first and initial_states is not None:           # the chain starts from the caller's state
            mine[0] = (torch.addcmul(mine[0][0], mine[0][1], _wide(initial_states)), mine[0][1])
        pairs, off = _exchange(chain, mine, R + 1, like)
        entering, final = states_entering(pairs, like)
        if first and initial_states is not None:
            entering[0] = _wide(initial_states)
        s_in = [None] * fo.n
        for pos, i in enumerate(order):
            s_in[i] = entering[off + pos].to(x.dtype)
        s_in_g = fo.per_group(s_in)
        res = [forward_final(be, o, xs[g], dts[g], A, Bs[g], Cs[g], D, zs[g], dt_bias, s_in_g[g]) for g in groups]
        out = fo.merge([r[0] for r in res], b)
        ctx.save_for_backward(x, dt, A, B, C, D, z, dt_bias, initial_states, *s_in_g, *[r[1] for r in res], *[r[3] for r in res],
                              *[p[1] for p in mine])
        ctx.chain, ctx.be, ctx.o, ctx.fo, ctx.order, ctx.R = chain, be, o, fo, order, R
        return out, final

    @staticmethod
    def backward(ctx, dout, dfinal):
        chain, be, o, fo, order, R = ctx.chain, ctx.be, ctx.o, ctx.fo, ctx.order, ctx.R
        x, dt, A, B, C, D, z, dt_bias, initial_states, *rest = ctx.saved_tensors
        ng = fo.groups
        s_in_g, out_x, saved, decs = rest[:ng], rest[ng:2 * ng], rest[2 * ng:3 * ng], rest[3 * ng:]
        b = x.shape[0]
        like = torch.zeros((b,) + tuple(s_in_g[0].shape[1:]), dtype=_wide(x).dtype, device=x.device)
        xs, dts, Bs, Cs, zs, gs = (fo.split(t) for t in (x, dt, B, C, z, dout))
        groups = range(ng)
        args = lambda g: (gs[g], xs[g], dts[g], A, Bs[g], Cs[g], D, zs[g], dt_bias, s_in_g[g], out_x[g], saved[g])
        G = fo.per_slice([_wide(backward_summary(be, o, *args(g))) for g in groups], b)
        mine = [(G[i], d) for i, d in zip(order, decs)]
        # the gradient of the final state travels with the pairs: the last rank in scan order appends it as one more
        # pair behind its slices (a = dfinal, dec = 1), the others an identity pair
        ones = torch.ones_like(decs[0])
        dfin = like if (dfinal is None or chain.pos != chain.world - 1) else _wide(dfinal)
        gpairs, off = _exchange(chain, mine + [(dfin, ones)], R + 2, like)
        leaving = grads_leaving(gpairs, None, like)
        ds_out = [None] * fo.n
        for pos, i in enumerate(order):
            ds_out[i] = leaving[off + pos]
        ds_g = fo.per_group(ds_out)
        res = [backward_final(be, o, *args(g), ds_g[g]) for g in groups]
        cat = lambda k: None if res[0][k] is None else fo.merge([r[k] for r in res], b)
        tot = lambda k: None if res[0][k] is None else sum(r[k] for r in res)
        dx, ddt, dB, dC, dz = cat(0), cat(1), cat(3), cat(4), cat(6)
        dA, dD, dbias = tot(2), tot(5), tot(7)
        ddt = ddt if ddt.dtype == dt.dtype else ddt.to(dt.dtype)
        if dbias is not None:
            dbias = (dbias if dt_bias.dim() == 2 else dbias.sum(dim=1)).to(dt_bias.dtype)
        dinit = None
        if initial_states is not None:
            if chain.pos == 0:
                dinit = fo.per_slice([r[8] for r in res], b)[order[0]].to(initial_states.dtype)
            else:
                dinit = torch.zeros_like(initial_states)
        return (None, None, None, None, dx, ddt, dA.to(A.dtype), dB.to(B.dtype), dC.to(C.dtype), None if dD is None else dD.to(D.dtype),
                None if dz is None else dz.to(z.dtype), dbias, dinit)


def _sliced(chain, R, x, dt, A, B, C, chunk_size, D, z, dt_bias, initial_states, dt_softplus, dt_limit, reverse, path, backend):
    o = Options(chunk_size, dt_softplus, dt_limit, reverse, path)
    return SlicedScanFn.apply(chain, backend, o, R, x, dt, A, B, C, D, z, dt_bias, initial_states)


def issm_scan_chunk_parallel(x, dt, A, B, C, chunk_size, D=None, z=None, dt_bias=None, initial_states=None,
                             dt_softplus=False, dt_limit=(0.0, float("inf")), return_final_states=False, reverse=False,
                             path="auto", slices=None, backend=KernelBackend):
    """`ISSM_chunk_scan_combined` for few, long sequences on one GPU: every sequence is cut into `slices` pieces that run
    as extra batch entries (two passes, see the module text).  `slices=None` picks the count from the sizes; with one
    slice this is the plain scan.  Same results as the plain scan up to the rounding of the carried states to the
    input dtype at the slice boundaries."""
    b, L, H, _ = x.shape
    R = pick_slices(b, H, L) if slices is None else int(slices)
    if R <= 1:
        return issm_combined.ISSM_chunk_scan_combined(x, dt, A, B, C, chunk_size, D=D, z=z, dt_bias=dt_bias, initial_states=initial_states,
                                                      dt_softplus=dt_softplus, dt_limit=dt_limit, return_final_states=return_final_states,
                                                      reverse=reverse, path=path)
    out, final = _sliced(Solo(), R, x, dt, A, B, C, chunk_size, D, z, dt_bias, initial_states, dt_softplus, dt_limit, reverse, path, backend)
    return (out, final) if return_final_states else out


def issm_scan_sequence_parallel(x, dt, A, B, C, chunk_size, D=None, z=None, dt_bias=None, initial_states=None,
                                dt_softplus=False, dt_limit=(0.0, float("inf")), reverse=False, path="auto", group=None,
                                slices=None, backend=KernelBackend):
    """`ISSM_chunk_scan_combined` for one sequence whose points are split over the ranks of `group`: rank r holds
    points [r L/R, (r + 1) L/R) of every tensor with a point axis (the parts may differ in length), and cuts its part
    into `slices` local slices (the same number on every rank; None picks it from the sizes of this rank, so pass a
    number when the parts differ much).  Returns (out of the local part, final_states of the WHOLE sequence, the same
    on every rank).  `initial_states` (the same on every rank, or None) enters at the first position; its gradient
    comes back there and is zero elsewhere.  The gradient of `final_states` is read on the rank that holds the end of
    the sequence in scan order.  dA / dD / ddt_bias are per-rank partial sums."""
    b, L, H, _ = x.shape
    world = dist.get_world_size(group)
    R = pick_slices(b, H, L, ranks=world) if slices is None else int(slices)
    return _sliced(RankChain(group, reverse), max(1, R), x, dt, A, B, C, chunk_size, D, z, dt_bias, initial_states, dt_softplus,
                   dt_limit, reverse, path, backend)
