"""tcgen05 building blocks (operand layouts, descriptors, TMEM row mapping) against torch.matmul, and the
bounded device-side wait; both through the test-only native library of tests/native."""
import ctypes as ct
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def selftest_lib():
    from tests.native import build
    path = build.LIB if os.path.exists(build.LIB) else build.build()
    return ct.CDLL(path)

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
    L = selftest_lib()
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


def test_bounded_wait_runs_out_and_the_device_stays_usable():
    """A wait on a barrier that nobody signals gives up after its poll limit: the kernel returns, bit 0 of the
    status word is set (what the ISSM kernels do when a copy or an MMA never completes), the Python layer turns
    that bit into an exception, and the next ordinary call on the same device is correct."""
    from dest3d_b200 import issm_combined
    from oracle import issm_oracle as O
    from tests import parity
    L = selftest_lib()
    L.issm_b200_selftest_bounded_wait.restype = ct.c_int
    issm_combined.device_status()                                   # clear
    word = issm_combined._status_word(torch.cuda.current_device())
    expired = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = L.issm_b200_selftest_bounded_wait(ct.c_uint32(1000), ct.c_void_p(word.data_ptr()), ct.c_void_p(expired.data_ptr()),
                                           ct.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    assert expired.item() == 1
    with pytest.raises(RuntimeError, match="bounded device-side wait"):
        issm_combined.raise_on_device_error()
    assert issm_combined.device_status() == 0                       # the exception cleared the word
    inp = O.make_inputs(1, 200, 2, 36, 256, seed=9, dtype=torch.bfloat16)
    opts = dict(dt_softplus=True, dt_limit=(1e-3, 1e-1))
    parity.compare(parity.cuda_run(inp, 256, opts, path="tensor"), parity.oracle_run(inp, 256, opts), torch.bfloat16)
    assert issm_combined.device_status() == 0


def test_expired_wait_surfaces_without_a_synchronising_check():
    """The default route: the status word is mirrored to pinned host memory behind the calls, and an ISSM call made after
    the failing kernels finished raises (within a few calls: one mirror copy is in flight at a time)."""
    from dest3d_b200 import issm_combined
    from oracle import issm_oracle as O
    from tests import parity
    L = selftest_lib()
    L.issm_b200_selftest_bounded_wait.restype = ct.c_int
    inp = O.make_inputs(1, 100, 2, 36, 256, seed=4, dtype=torch.bfloat16)
    opts = dict(dt_softplus=True, dt_limit=(1e-3, 1e-1), return_final=False, dfinal=False)
    issm_combined.device_status()                                   # clear
    parity.cuda_run(inp, 256, opts, path="tensor")                  # a healthy call: mirror copy in flight
    word = issm_combined._status_word(torch.cuda.current_device())
    expired = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert L.issm_b200_selftest_bounded_wait(ct.c_uint32(1000), ct.c_void_p(word.data_ptr()), ct.c_void_p(expired.data_ptr()),
                                             ct.c_void_p(torch.cuda.current_stream().cuda_stream)) == 0
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="bounded device-side wait"):
        for _ in range(4):
            parity.cuda_run(inp, 256, opts, path="tensor")
            torch.cuda.synchronize()
    assert issm_combined.device_status() == 0                       # raising cleared the word
    parity.cuda_run(inp, 256, opts, path="tensor")                  # and the device goes on working
    torch.cuda.synchronize()
    assert issm_combined.device_status() & 1 == 0
