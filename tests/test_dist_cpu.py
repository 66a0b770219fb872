"""Multi-rank host logic on CPU ranks (gloo, world_size 2): sharding, the packed parameter-gradient
all-reduce, max-over-ranks timing, and a host-injected failure (a rank that never joins)."""
import os
import socket
from datetime import timedelta

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from dest3d_b200.dist import PackedParamGrads, max_over_ranks, shard_samples


def test_shard_samples_cover_everything():
    for gb in (1, 7, 16, 64):
        for ws in (1, 2, 3, 8):
            seen = []
            for r in range(ws):
                seen += list(shard_samples(gb, ws, r))
            assert seen == list(range(gb))
    assert [len(shard_samples(64, 8, r)) for r in range(8)] == [8] * 8
    assert [len(shard_samples(7, 2, r)) for r in range(2)] == [4, 3]
    with pytest.raises(ValueError):
        shard_samples(4, 2, 2)


def test_packed_views_alias_flat_buffer():
    p = PackedParamGrads({"dA": (8, 256), "ddt_bias": (8, 256), "dD": (8,), "dW": (288,)}, "cpu")
    assert p.flat.numel() == 2 * 8 * 256 + 8 + 288 == 4392
    p.load({"dA": torch.ones(8, 256), "dD": torch.arange(8.0)})
    assert p.flat[:2048].sum() == 2048 and p.views["ddt_bias"].abs().sum() == 0
    assert torch.equal(p.flat[4096:4104], torch.arange(8.0))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, mode, ret):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    if mode == "absent" and rank == 1:
        ret[rank] = "stayed away"
        return                                  # host-injected failure: this rank never joins
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=5))
    except Exception as e:                      # the surviving rank must get an error, not hang
        ret[rank] = f"error: {type(e).__name__}"
        return
    shapes = {"dA": (2, 4), "ddt_bias": (2, 4), "dD": (2,)}
    mine = shard_samples(5, world, rank)
    grads = {k: torch.full(s, float(sum(mine) + 1)) for k, s in shapes.items()}
    packed = PackedParamGrads(shapes, "cpu").load(grads).all_reduce()
    expect = float(sum(sum(shard_samples(5, world, r)) + 1 for r in range(world)))
    ok = all(torch.all(v == expect).item() for v in packed.views.values())
    t = max_over_ranks(1.0 + rank, "cpu")
    ret[rank] = "ok" if ok and t == float(world) else f"bad: {packed.flat.tolist()} {t}"
    dist.destroy_process_group()


def _run(mode):
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, mode, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert not p.is_alive(), "worker hung"
    return dict(ret)


def test_two_rank_all_reduce_gloo():
    assert _run("normal") == {0: "ok", 1: "ok"}


def test_rank_that_never_joins_is_an_error_not_a_hang():
    ret = _run("absent")
    assert ret[1] == "stayed away" and ret[0].startswith("error")
