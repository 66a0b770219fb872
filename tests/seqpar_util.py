"""Test helpers for the sequence-parallel mode: an oracle-backed stand-in for the kernel backend (same call
signatures as dest3d_b200.issm_combined.issm_fwd / issm_bwd, float64 on the CPU) and slicing of a parity input."""
import torch

from oracle import issm_oracle as O

POINT_AXIS = ("x", "dt", "B", "C", "z", "dout")


class OracleBackend:
    """issm_fwd / issm_bwd semantics on top of the differentiable oracle (for CPU ranks; checker only)."""

    @staticmethod
    def decay(dt, A, dt_bias, o):
        """exp(A * sum of the transformed dt over the slice), (b, H, 1, N)."""
        v = O.dt_transform(dt.double(), None if dt_bias is None else dt_bias.double(), o.dt_softplus, o.dt_limit)
        return torch.exp(A.double() * v.sum(dim=1)).unsqueeze(2)

    @staticmethod
    def _run(x, dt, A, B, C, chunk_size, D, z, dt_bias, init, dt_softplus, dt_limit, reverse, grad):
        t = dict(x=x, dt=dt, A=A, B=B, C=C, D=D, z=z, dt_bias=dt_bias, init=init)
        t = {k: (None if v is None else v.detach().double().requires_grad_(grad)) for k, v in t.items()}
        out, fin = O.issm_scan_chunked(t["x"], t["dt"], t["A"], t["B"], t["C"], chunk_size, D=t["D"], z=t["z"], dt_bias=t["dt_bias"],
                                       initial_states=t["init"], dt_softplus=dt_softplus, dt_limit=dt_limit, reverse=reverse,
                                       compute_dtype=torch.float64)
        return t, out, fin

    @staticmethod
    def fwd(x, dt, A, B, C, chunk_size, D=None, z=None, dt_bias=None, initial_states=None, dt_softplus=False,
            dt_limit=(0.0, float("inf")), reverse=False, path="auto", want_final=True, save_states=False):
        with torch.no_grad():
            _, out, fin = OracleBackend._run(x, dt, A, B, C, chunk_size, D, z, dt_bias, initial_states, dt_softplus, dt_limit, reverse, False)
        return (out, None, fin, None) if save_states else (out, None, fin)

    @staticmethod
    def bwd(dout, x, dt, A, B, C, out_x, chunk_size, D=None, z=None, dt_bias=None, initial_states=None, dfinal_states=None,
            dt_softplus=False, dt_limit=(0.0, float("inf")), reverse=False, path="auto", saved_states=None):
        with torch.enable_grad():
            t, out, fin = OracleBackend._run(x, dt, A, B, C, chunk_size, D, z, dt_bias, initial_states, dt_softplus, dt_limit, reverse, True)
            loss = (out * dout.double()).sum()
            if dfinal_states is not None:
                loss = loss + (fin * dfinal_states.double()).sum()
            loss.backward()
        g = lambda k: None if t[k] is None else t[k].grad
        return g("x"), g("dt"), g("A"), g("B"), g("C"), g("D"), g("z"), g("dt_bias"), g("init")


def split_points(inp, parts):
    """Cut the point-axis tensors of a parity input into `parts` contiguous slices of (nearly) equal length."""
    L = inp["x"].shape[1]
    edges = [L * i // parts for i in range(parts + 1)]
    out = []
    for i in range(parts):
        out.append({k: inp[k][:, edges[i]:edges[i + 1]] for k in POINT_AXIS if inp.get(k) is not None})
    return out
