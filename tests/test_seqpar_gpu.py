"""One sequence cut into slices, on the CUDA kernels: slices folded into the batch axis on one GPU against the oracle
on the WHOLE sequence; and, where two GPUs are visible, the parts of two ranks chained over NCCL."""
import os
import socket

import pytest
import torch

from oracle import issm_oracle as O
from tests import parity
from tests.seqpar_util import split_points

pytestmark = pytest.mark.gpu
OPTS = dict(dt_softplus=True, dt_limit=(1e-3, 1e-1))


@pytest.mark.parametrize("dtype,path,L,slices,reverse", [
    (torch.bfloat16, "tensor", 1000, 4, False), (torch.bfloat16, "tensor", 1009, 4, True), (torch.bfloat16, "tensor", 4096, 16, False),
    (torch.float32, "simt", 300, 3, True)])
def test_chunk_parallel_on_one_gpu_matches_whole_sequence(dtype, path, L, slices, reverse):
    """Slices folded into the batch axis (with and without a ragged tail), through the public call, batch of 2."""
    from dest3d_b200.seqpar import issm_scan_chunk_parallel
    N = 256 if path == "tensor" else 64
    inp = O.make_inputs(2, L, 2, 36, N, seed=17, dtype=dtype)
    ref = parity.oracle_run_sliced(inp, 64, dict(OPTS, reverse=reverse))
    names = ("x", "dt", "A", "B", "C", "D", "z", "dt_bias", "initial_states")
    lv = {k: inp[k].cuda().requires_grad_() for k in names}
    out, fin = issm_scan_chunk_parallel(lv["x"], lv["dt"], lv["A"], lv["B"], lv["C"], 64, D=lv["D"], z=lv["z"], dt_bias=lv["dt_bias"],
                                        initial_states=lv["initial_states"], return_final_states=True, reverse=reverse, path=path,
                                        slices=slices, **OPTS)
    ((out.float() * inp["dout"].cuda().float()).sum() + (fin * inp["dfinal"].cuda()).sum()).backward()
    got = {"out": out.detach(), "final": fin.detach()}
    got.update({"d" + k: lv[k].grad for k in names})
    print(parity.format_report(parity.compare(got, ref, dtype)))


def test_slices_keyword_of_the_public_call():
    from dest3d_b200 import ISSM_chunk_scan_combined
    inp = O.make_inputs(1, 1024, 2, 36, 256, seed=23, dtype=torch.bfloat16)
    t = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in inp.items()}
    args = (t["x"], t["dt"], t["A"], t["B"], t["C"], 64)
    kw = dict(D=t["D"], z=t["z"], dt_bias=t["dt_bias"], initial_states=t["initial_states"], return_final_states=True, **OPTS)
    from dest3d_b200 import _lib
    n0 = _lib.launch_count()
    y1, s1 = ISSM_chunk_scan_combined(*args, **kw)
    n1 = _lib.launch_count()
    y4, s4 = ISSM_chunk_scan_combined(*args, slices=4, **kw)
    assert _lib.launch_count() - n1 > n1 - n0               # two passes plus the decay sums: the sliced route was taken
    ya, sa = ISSM_chunk_scan_combined(*args, slices="auto", **kw)          # 2 heads x 1 sample: cut into 2 (512 points each)
    for y, s in ((y4, s4), (ya, sa)):
        torch.testing.assert_close(y.float(), y1.float(), rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(s, s1, rtol=2e-2, atol=2e-2)


def test_automatic_slice_count_falls_back_to_the_plain_scan():
    from dest3d_b200.seqpar import issm_scan_chunk_parallel
    inp = O.make_inputs(2, 300, 8, 36, 256, seed=2, dtype=torch.bfloat16)
    t = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in inp.items()}
    a = issm_scan_chunk_parallel(t["x"], t["dt"], t["A"], t["B"], t["C"], 64, D=t["D"], dt_bias=t["dt_bias"], **OPTS)
    from dest3d_b200 import ISSM_chunk_scan_combined
    assert torch.equal(a, ISSM_chunk_scan_combined(t["x"], t["dt"], t["A"], t["B"], t["C"], 64, D=t["D"], dt_bias=t["dt_bias"], **OPTS))


def _nccl_worker(rank, world, port, ret):
    import torch.distributed as dist
    from dest3d_b200.seqpar import issm_scan_sequence_parallel
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    inp = O.make_inputs(1, 2000, 2, 36, 256, seed=13, dtype=torch.bfloat16)
    mine = {k: v.cuda() for k, v in split_points(inp, world)[rank].items()}
    leaves = {k: v.clone().requires_grad_() for k, v in mine.items() if k != "dout"}
    par = {k: inp[k].cuda().requires_grad_() for k in ("A", "D", "dt_bias", "initial_states")}
    out, fin = issm_scan_sequence_parallel(leaves["x"], leaves["dt"], par["A"], leaves["B"], leaves["C"], 64, D=par["D"], z=leaves["z"],
                                           dt_bias=par["dt_bias"], initial_states=par["initial_states"], path="tensor", slices=3, **OPTS)
    ((out.float() * mine["dout"].float()).sum() + (fin * inp["dfinal"].cuda()).sum()).backward()
    torch.cuda.synchronize()
    res = {"out": out.detach().cpu(), "final": fin.detach().cpu()}
    res.update({"d" + k: v.grad.cpu() for k, v in leaves.items()})
    res.update({"d" + k: v.grad.cpu() for k, v in par.items()})
    ret[rank] = res
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpus_over_nccl():
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_nccl_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    inp = O.make_inputs(1, 2000, 2, 36, 256, seed=13, dtype=torch.bfloat16)
    ref = parity.oracle_run(inp, 64, OPTS)
    got = {k: torch.cat([ret[r][k] for r in range(2)], dim=1) for k in ("out", "dx", "ddt", "dB", "dC", "dz")}
    got.update({k: sum(ret[r][k].float() for r in range(2)) for k in ("dA", "dD", "ddt_bias")})
    got.update(final=ret[1]["final"], dinitial_states=ret[0]["dinitial_states"])
    assert torch.equal(ret[0]["final"], ret[1]["final"])
    print(parity.format_report(parity.compare(got, ref, torch.bfloat16)))
