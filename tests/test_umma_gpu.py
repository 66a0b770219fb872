"""tcgen05 building blocks (operand layouts, descriptors, TMEM row mapping) against torch.matmul."""
import ctypes as ct

import pytest
import torch

pytestmark = pytest.mark.gpu

CONFIGS = [
    # M, N, K, kindA, kindB   (kind 0 = 128-byte swizzle K-major, 1 = interleaved core matrices)
    (128, 64, 64, 0, 0), (128, 48, 64, 0, 0), (64, 64, 256, 0, 0), (64, 48, 256, 0, 0), (64, 48, 64, 0, 0),
    (128, 64, 48, 1, 1), (128, 64, 48, 1, 0), (128, 64, 48, 0, 0), (64, 64, 48, 0, 0), (128, 48, 64, 0, 1),
    (128, 256, 64, 0, 0), (128, 64, 16, 1, 1),
    # kind 2 = MN-major operand in 128-byte-swizzle storage (the transposed tile's K-major storage)
    (128, 64, 64, 2, 0), (128, 64, 64, 0, 2), (128, 48, 64, 2, 2), (64, 64, 64, 2, 2), (64, 48, 256, 0, 2),
    (128, 64, 48, 2, 0), (64, 48, 64, 2, 2),
]


@pytest.mark.parametrize("cfg", CONFIGS, ids=[f"M{c[0]}N{c[1]}K{c[2]}a{c[3]}b{c[4]}" for c in CONFIGS])
def test_umma_matches_matmul(cfg):
    from dest3d_b200 import _lib
    L = _lib.lib()
    M, N, K, ka, kb = cfg
    g = torch.Generator().manual_seed(M + N + K)
    A = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    B = torch.randn(N, K, generator=g).to(torch.bfloat16).cuda()
    D = torch.full((M, N), float("nan"), device="cuda")
    Draw = torch.zeros(128, N, device="cuda")
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    L.issm_b200_selftest_umma.restype = ct.c_int
    rc = L.issm_b200_selftest_umma(M, N, K, ka, kb, ct.c_void_p(A.data_ptr()), ct.c_void_p(B.data_ptr()),
                                   ct.c_void_p(D.data_ptr()), ct.c_void_p(Draw.data_ptr()), ct.c_void_p(st.data_ptr()),
                                   ct.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    assert st.item() == 0, "bounded wait on the MMA completion barrier expired"
    ref = A.float() @ B.float().t()
    err = (D - ref).abs().max().item()
    if not err < 1e-2:
        # help the diagnosis: which raw TMEM lane holds which reference row?
        hits = []
        for lane in range(128):
            d = (Draw[lane][None, :] - ref).abs().max(dim=1).values
            r = int(d.argmin())
            hits.append((lane, r, float(d[r])))
        print("lane -> best matching row (err):", [(l, r, round(e, 3)) for l, r, e in hits if e < 1e-2][:40])
    assert err < 1e-2, f"max abs err {err}"
