"""The benchmark's named configurations as parity cases (at sizes the oracle finishes in seconds):
C1 = bidirectional ISSM layer + z-gated RMSNorm, forward and backward (models/dest_module.py:565-579);
C2 = stacked forward-only layers whose final states seed the next layer's initial states."""
import pytest
import torch

from oracle import issm_oracle as O
from tests import parity

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,path", [(torch.bfloat16, "tensor"), (torch.float32, "simt")], ids=["bf16_tensor", "f32_simt"])
def test_c1_bidirectional_layer_with_gated_rmsnorm(dtype, path):
    from dest3d_b200 import RMSNorm, issm_bidirectional_scan
    b, L, H, P, N, Q = 2, 200, 8, 36, 256, 256
    inp = O.make_inputs(b, L, H, P, N, seed=21, dtype=dtype)
    inp2 = O.make_inputs(b, L, H, P, N, seed=22, dtype=dtype)
    g = torch.Generator().manual_seed(5)
    w = 1 + 0.02 * torch.randn(H * P, generator=g)
    dout = torch.randn(b, L, H * P, generator=g).to(dtype)
    names = ["x", "xb", "dt", "A", "B", "C", "Bb", "Cb", "D", "dt_bias", "init", "z", "w"]
    vals = [inp["x"], inp2["x"], inp["dt"], inp["A"], inp["B"], inp["C"], inp2["B"], inp2["C"], inp["D"],
            inp["dt_bias"], inp["initial_states"], inp["z"], w]
    # oracle in float64
    R = {k: v.detach().double().requires_grad_() for k, v in zip(names, vals)}
    y, fin = O.issm_scan_bidirectional(R["x"], R["xb"], R["dt"], R["A"], R["B"], R["C"], R["Bb"], R["Cb"], Q, D=R["D"],
                                       dt_bias=R["dt_bias"], initial_states=R["init"], dt_softplus=True,
                                       dt_limit=(1e-3, 1e-1), compute_dtype=torch.float64)
    key = y.reshape(b, L, H * P)
    xg = key * torch.nn.functional.silu(R["z"].reshape(b, L, H * P))
    yn = xg * torch.rsqrt(xg.square().mean(-1, keepdim=True) + 1e-5) * R["w"]
    ((yn * dout.double()).sum() + (fin * inp["dfinal"].double()).sum()).backward()
    # CUDA path
    Cc = {k: v.detach().clone().cuda().requires_grad_() for k, v in zip(names, vals)}
    norm = RMSNorm(H * P, eps=1e-5, norm_before_gate=False, device="cuda")
    with torch.no_grad():
        norm.weight.copy_(w)
    y2, fin2 = issm_bidirectional_scan(Cc["x"], Cc["xb"], Cc["dt"], Cc["A"], Cc["B"], Cc["C"], Cc["Bb"], Cc["Cb"], Q,
                                       D=Cc["D"], dt_bias=Cc["dt_bias"], initial_states=Cc["init"], dt_softplus=True,
                                       dt_limit=(1e-3, 1e-1), path=path)
    yn2 = norm(y2.reshape(b, L, H * P), Cc["z"].reshape(b, L, H * P))
    ((yn2.float() * dout.cuda().float()).sum() + (fin2 * inp["dfinal"].cuda()).sum()).backward()
    # the scan's outputs literally; what passes through the norm (which divides by the row RMS and so amplifies the
    # error its input carries) relative to the reference tensor's largest magnitude
    parity.close(y2, y, dtype, "out", literal=False)       # average of two scans that can cancel (each is checked literally elsewhere)
    parity.close(fin2, fin, dtype, "final")
    parity.close(yn2, yn, dtype, "normed out", literal=False)
    parity.close(norm.weight.grad, R["w"].grad, dtype, "dW")
    for k in names[:-1]:
        parity.close(Cc[k].grad, R[k].grad, dtype, "d" + k, literal=False)


@pytest.mark.parametrize("dtype,path,N,Q", [(torch.bfloat16, "tensor", 256, 128), (torch.float32, "simt", 512, 128),
                                             (torch.bfloat16, "simt", 512, 128), (torch.bfloat16, "tensor", 512, 128)],
                         ids=["bf16_tensor_n256", "f32_n512", "bf16_n512", "bf16_tensor_n512"])
def test_c2_stacked_layers_chain_states(dtype, path, N, Q):
    from dest3d_b200 import ISSM_chunk_scan_combined
    b, L, H, P, layers = 1, 192, 2, 36, 3
    init = torch.randn(b, H, P, N, generator=torch.Generator().manual_seed(3)) / 16
    s_ref, s_gpu = init.double(), init.to(dtype).cuda()
    for k in range(layers):
        inp = O.make_inputs(b, L, H, P, N, seed=30 + k, dtype=dtype)
        kw = dict(D=inp["D"], dt_bias=inp["dt_bias"], dt_softplus=True, dt_limit=(1e-3, 1e-1))
        yr, s_ref = O.issm_scan_chunked(inp["x"], inp["dt"], inp["A"], inp["B"], inp["C"], Q, initial_states=s_ref.to(dtype),
                                        compute_dtype=torch.float64, **kw)
        c = {k2: (v.cuda() if torch.is_tensor(v) else v) for k2, v in inp.items()}
        yg, s_next = ISSM_chunk_scan_combined(c["x"], c["dt"], c["A"], c["B"], c["C"], Q, D=c["D"], dt_bias=c["dt_bias"],
                                              initial_states=s_gpu, dt_softplus=True, dt_limit=(1e-3, 1e-1),
                                              return_final_states=True, path=path)
        parity.close(yg, yr, dtype, f"layer {k} out")
        parity.close(s_next, s_ref, dtype, f"layer {k} final")
        s_gpu = s_next.to(dtype)            # the next layer starts from this layer's final states
        s_ref = s_gpu.double().cpu()        # keep the two chains on identical (rounded) states
