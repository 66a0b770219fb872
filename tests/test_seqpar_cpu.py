"""Sequence-parallel mode on CPU ranks (gloo, world_size 2 and 3) with the oracle as the scan backend: outputs, final
state and every gradient of the split run equal the oracle on the whole sequence."""
import os
import socket
from datetime import timedelta

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import issm_oracle as O
from tests import parity
from tests.seqpar_util import OracleBackend, split_points


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, reverse, slices, ret):
    from dest3d_b200.seqpar import issm_scan_sequence_parallel
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=60))
    torch.set_num_threads(2)
    inp = O.make_inputs(2, 150, 2, 4, 8, seed=3, dtype=torch.float64)
    mine = split_points(inp, world)[rank]
    leaves = {k: v.clone().requires_grad_() for k, v in mine.items() if k != "dout"}
    par = {k: inp[k].double().clone().requires_grad_() for k in ("A", "D", "dt_bias", "initial_states")}
    out, fin = issm_scan_sequence_parallel(leaves["x"], leaves["dt"], par["A"], leaves["B"], leaves["C"], 32, D=par["D"], z=leaves["z"],
                                           dt_bias=par["dt_bias"], initial_states=par["initial_states"], dt_softplus=True,
                                           dt_limit=(1e-3, 1e-1), reverse=reverse, slices=slices, backend=OracleBackend)
    # the final state's gradient is fed on every rank; only the copy at the end of the scan order may count
    (out * mine["dout"]).sum().add((fin * inp["dfinal"].double()).sum()).backward()
    res = {"out": out.detach(), "final": fin.detach()}
    res.update({"d" + k: v.grad for k, v in leaves.items()})
    res.update({"d" + k: v.grad for k, v in par.items()})
    ret[rank] = res
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,reverse,slices", [(2, False, 1), (2, True, 3), (3, False, 2)])
def test_split_sequence_matches_whole_sequence(world, reverse, slices):
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, reverse, slices, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
        assert p.exitcode == 0
    inp = O.make_inputs(2, 150, 2, 4, 8, seed=3, dtype=torch.float64)
    ref = parity.oracle_run(inp, 32, dict(dt_softplus=True, dt_limit=(1e-3, 1e-1), reverse=reverse))
    tol = dict(rtol=1e-9, atol=1e-11)
    for k in ("out", "dx", "ddt", "dB", "dC", "dz"):
        torch.testing.assert_close(torch.cat([ret[r][k] for r in range(world)], dim=1), ref[k], **tol)
    for k in ("dA", "dD", "ddt_bias"):                      # per-rank partial sums
        torch.testing.assert_close(sum(ret[r][k] for r in range(world)), ref[k], **tol)
    first = world - 1 if reverse else 0
    for r in range(world):
        torch.testing.assert_close(ret[r]["final"], ref["final"], **tol)
        if r == first:
            torch.testing.assert_close(ret[r]["dinitial_states"], ref["dinitial_states"], **tol)
        else:
            assert ret[r]["dinitial_states"].abs().max() == 0


@pytest.mark.parametrize("L,slices,reverse,with_init", [(150, 3, False, True), (157, 4, True, True), (128, 2, False, False), (90, 5, True, False)])
def test_chunk_parallel_folding_matches_whole_sequence(L, slices, reverse, with_init):
    """The single-GPU variant (slices folded into the batch axis) with the oracle as backend, float64: exact."""
    from dest3d_b200.seqpar import issm_scan_chunk_parallel
    inp = O.make_inputs(2, L, 2, 4, 8, seed=4, dtype=torch.float64, with_init=with_init)
    inp = {k: (v.double() if torch.is_tensor(v) else v) for k, v in inp.items()}
    ref = parity.oracle_run(inp, 32, dict(dt_softplus=True, dt_limit=(1e-3, 1e-1), reverse=reverse))
    names = ("x", "dt", "A", "B", "C", "D", "z", "dt_bias") + (("initial_states",) if with_init else ())
    lv = {k: inp[k].clone().requires_grad_() for k in names}
    out, fin = issm_scan_chunk_parallel(lv["x"], lv["dt"], lv["A"], lv["B"], lv["C"], 32, D=lv["D"], z=lv["z"], dt_bias=lv["dt_bias"],
                                        initial_states=lv.get("initial_states"), dt_softplus=True, dt_limit=(1e-3, 1e-1),
                                        return_final_states=True, reverse=reverse, slices=slices, backend=OracleBackend)
    ((out * inp["dout"]).sum() + (fin * inp["dfinal"]).sum()).backward()
    tol = dict(rtol=1e-9, atol=1e-11)
    torch.testing.assert_close(out.detach(), ref["out"], **tol)
    torch.testing.assert_close(fin.detach(), ref["final"], **tol)
    for k in names:
        torch.testing.assert_close(lv[k].grad, ref["d" + k], **tol)


def test_slice_count_choice():
    from dest3d_b200.seqpar import _layout, pick_slices
    assert pick_slices(1, 8, 40000) == 19 and pick_slices(16, 8, 40000) == 1 and pick_slices(8, 8, 1024) == 1
    assert pick_slices(1, 8, 1200) == 2                      # never below 512 points per slice
    assert _layout(40000, 16) == (2500, 16, 0) and _layout(1009, 4) == (253, 3, 250)
    for L in (64, 100, 1009, 40000):
        for R in (2, 3, 7, 19):
            lr, rf, tail = _layout(L, R)
            assert lr * rf + tail == L and tail < lr and rf >= 1
