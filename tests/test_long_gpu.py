"""Parity of the tensor-core path at the benchmark's own sequence length and configurations.

The benchmark walks 625 blocks of 64 points per (sample, head) stream: the running state is re-rounded to
bf16 as an MMA operand every block, the backward consumes the bf16 block-entry states saved by the forward
and rescales the state gradient once per block, and the per-head dB / dC partials are rounded to bf16 before
the head sum.  These cases check that none of this drifts over a long walk:
  * L = 40000 (the benchmark's length): out and final states, both scan directions, against the float64
    step-by-step recurrence (memory O(b H P N));
  * L = 8229 (128 full blocks and a 37-point tail): out, final states and every gradient against the float64
    chunked oracle evaluated one (sample, head) stream at a time;
  * the detector-sized layer (batch 8, L = 1024, bidirectional, z-gated RMSNorm over all heads) at full size,
    one sample at a time.
Inputs follow the benchmark's distributions (oracle.make_inputs)."""
import pytest
import torch

from oracle import issm_oracle as O
from tests import parity

pytestmark = pytest.mark.gpu
OPTS = dict(dt_softplus=True, dt_limit=(1e-3, 1e-1))


@pytest.mark.parametrize("reverse", [False, True], ids=["forward_scan", "reversed_scan"])
def test_benchmark_length_forward_against_recurrence(reverse):
    from dest3d_b200 import issm_fwd
    from dest3d_b200.issm_combined import device_status
    b, L, H, P, N, Q = 1, 40000, 2, 36, 256, 256
    inp = O.make_inputs(b, L, H, P, N, seed=40 + int(reverse), dtype=torch.bfloat16)
    with torch.no_grad():
        ref_out, ref_fin = O.issm_scan_sequential(inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"], Q, D=inp["D"], z=inp["z"],
                                                  dt_bias=inp["dt_bias"], initial_states=inp["initial_states"],
                                                  reverse=reverse, compute_dtype=torch.float64, **OPTS)
    c = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in inp.items()}
    device_status()
    out, out_x, fin = issm_fwd(c["x"], c["dt"], c["A"], c["B"], c["C"], Q, D=c["D"], z=c["z"], dt_bias=c["dt_bias"],
                               initial_states=c["initial_states"], reverse=reverse, path="tensor", **OPTS)
    assert device_status() == 0
    rep = []
    parity.close(out, ref_out, torch.bfloat16, "out", rep)
    parity.close(fin, ref_fin, torch.bfloat16, "final", rep)
    print("L=40000", "reversed" if reverse else "forward", parity.format_report(rep))


@pytest.mark.parametrize("reverse", [False, True], ids=["forward_scan", "reversed_scan"])
def test_long_walk_all_gradients(reverse):
    """128 full blocks and a tail through the forward and backward tensor-core kernels."""
    from dest3d_b200.issm_combined import device_status
    b, L, H, P, N, Q = 1, 8229, 2, 36, 256, 256
    inp = O.make_inputs(b, L, H, P, N, seed=50 + int(reverse), dtype=torch.bfloat16)
    opts = dict(OPTS, reverse=reverse)
    ref = parity.oracle_run_sliced(inp, 64, opts)           # the oracle's chunk length does not change its result
    device_status()
    got = parity.cuda_run(inp, Q, opts, path="tensor")
    assert device_status() == 0
    rep = parity.compare(got, ref, torch.bfloat16)
    print("L=8229", "reversed" if reverse else "forward", parity.format_report(rep))


def test_detector_layer_full_size():
    """Batch 8 x L 1024 x 8 heads x 36, 256 states, chunk 256: the bidirectional layer followed by the z-gated
    RMSNorm over all 288 features (models/dest_module.py:565-579), forward and backward."""
    from dest3d_b200 import RMSNorm, issm_bidirectional_scan
    b, L, H, P, N, Q = 8, 1024, 8, 36, 256, 256
    dtype = torch.bfloat16
    inp = O.make_inputs(b, L, H, P, N, seed=61, dtype=dtype)
    inp2 = O.make_inputs(b, L, H, P, N, seed=62, dtype=dtype)
    g = torch.Generator().manual_seed(5)
    w = 1 + 0.02 * torch.randn(H * P, generator=g)
    dout = torch.randn(b, L, H * P, generator=g).to(dtype)
    names = ["x", "xb", "dt", "A", "B", "C", "Bb", "Cb", "D", "dt_bias", "init", "z", "w"]
    vals = [inp["x"], inp2["x"], inp["dt"], inp["A"], inp["B"], inp["C"], inp2["B"], inp2["C"], inp["D"],
            inp["dt_bias"], inp["initial_states"], inp["z"], w]
    per_sample = {"x", "xb", "dt", "B", "C", "Bb", "Cb", "init", "z"}
    ref_grad = {k: torch.zeros(v.shape, dtype=torch.float64) for k, v in zip(names, vals)}
    ref_y = torch.zeros(b, L, H * P, dtype=torch.float64)
    ref_key = torch.zeros(b, L, H, P, dtype=torch.float64)
    ref_mag = torch.zeros(b, L, H, P, dtype=torch.float64)       # 0.5 (|y_forward| + |y_reversed|): the directions can cancel
    ref_fin = torch.zeros(b, H, P, N, dtype=torch.float64)
    for i in range(b):                                        # oracle in float64, one sample at a time
        R = {k: (v[i:i + 1] if k in per_sample else v).detach().double().requires_grad_() for k, v in zip(names, vals)}
        skw = dict(D=R["D"], dt_bias=R["dt_bias"], initial_states=R["init"], dt_softplus=True, dt_limit=(1e-3, 1e-1),
                   compute_dtype=torch.float64)
        yf, sf = O.issm_scan_chunked(R["x"], R["dt"], R["A"], R["B"], R["C"], 64, **skw)
        yb, sb = O.issm_scan_chunked(R["xb"], R["dt"], R["A"], R["Bb"], R["Cb"], 64, reverse=True, **skw)
        y, fin = (yf + yb) * 0.5, (sf + sb) * 0.5             # models/dest_module.py:574-575
        ref_mag[i:i + 1] = 0.5 * (yf.detach().abs() + yb.detach().abs())
        xg = y.reshape(1, L, H * P) * torch.nn.functional.silu(R["z"].reshape(1, L, H * P))
        yn = xg * torch.rsqrt(xg.square().mean(-1, keepdim=True) + 1e-5) * R["w"]
        ((yn * dout[i:i + 1].double()).sum() + (fin * inp["dfinal"][i:i + 1].double()).sum()).backward()
        ref_y[i:i + 1], ref_fin[i:i + 1], ref_key[i:i + 1] = yn.detach(), fin.detach(), y.detach()
        for k in names:
            if k in per_sample:
                ref_grad[k][i:i + 1] = R[k].grad
            else:
                ref_grad[k] += R[k].grad
    Cc = {k: v.detach().clone().cuda().requires_grad_() for k, v in zip(names, vals)}
    norm = RMSNorm(H * P, eps=1e-5, norm_before_gate=False, device="cuda")
    with torch.no_grad():
        norm.weight.copy_(w)
    y2, fin2 = issm_bidirectional_scan(Cc["x"], Cc["xb"], Cc["dt"], Cc["A"], Cc["B"], Cc["C"], Cc["Bb"], Cc["Cb"], Q,
                                       D=Cc["D"], dt_bias=Cc["dt_bias"], initial_states=Cc["init"], dt_softplus=True,
                                       dt_limit=(1e-3, 1e-1), path="tensor")
    yn2 = norm(y2.reshape(b, L, H * P), Cc["z"].reshape(b, L, H * P))
    ((yn2.float() * dout.cuda().float()).sum() + (fin2 * inp["dfinal"].cuda()).sum()).backward()
    # The combined key is the average of two scans that may cancel: each direction is allowed its own literal
    # tolerance (atol + rtol |y_direction|), and the bf16 rounding of the combined value comes on top.
    # The norm divides each row by its RMS (rows with a
    # small RMS amplify whatever error their input carries, here up to ~10x), so (a) the norm is checked on its own,
    # literally, against the float64 formula applied to the key the GPU scan produced, and (b) the end-to-end
    # output and the gradients, which all pass through the norm's backward, are compared relative to the largest
    # magnitude of the reference tensor (the report prints that scale).
    rep = []
    err = (y2.detach().double().cpu() - ref_key).abs()
    bound = 1e-2 + 1e-2 * ref_mag + 2.0 ** -8 * ref_key.abs()
    worst = (err / bound).max().item()
    rep.append(("out", err.max().item(), 1.0, worst))
    assert worst <= 1.0, f"out: max err {err.max().item():.3e} exceeds the two directions' tolerance x{worst:.2f}"
    parity.close(fin2, ref_fin, dtype, "final", rep)
    kg = y2.detach().double().cpu().reshape(b, L, H * P) * torch.nn.functional.silu(inp["z"].double().reshape(b, L, H * P))
    parity.close(yn2, kg * torch.rsqrt(kg.square().mean(-1, keepdim=True) + 1e-5) * w.double(), dtype, "norm of the GPU key", rep, literal=True)
    parity.close(yn2, ref_y, dtype, "normed out", rep, literal=False)
    parity.close(norm.weight.grad, ref_grad["w"], dtype, "dW", rep)
    for k in names[:-1]:
        parity.close(Cc[k].grad, ref_grad[k], dtype, "d" + k, rep, literal=False)
    print("detector layer b8 L1024:", parity.format_report(rep))
