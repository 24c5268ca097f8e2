"""The multi-GPU path (independent replicas, no data-path collective) with two
gloo ranks on the CPU: row sharding and the aggregation of per-rank results."""

import os
import sys
from pathlib import Path

import pytest
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def _worker(rank, world, port, out):
    sys.path.insert(0, str(ROOT))
    import __graft_entry__  # noqa: F401
    import torch.distributed as dist
    from dfb_b200 import replicas

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rows = replicas.shard_rows(5, rank, world)
        replicas.barrier(dist)
        tokens, slowest = replicas.aggregate(dist, tokens=len(rows) * 10, elapsed_ms=3.0 + rank, device="cpu")
        out[rank] = (list(rows), tokens, slowest)
    finally:
        dist.destroy_process_group()


def test_two_rank_aggregation():
    ctx = mp.get_context("spawn")
    out = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, 2, 29733, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert out[0][0] == [0, 1, 2] and out[1][0] == [3, 4]
    for r in range(2):
        assert out[r][1] == 50          # tokens of both ranks
        assert out[r][2] == 4.0         # the slowest rank sets the time


def test_shard_rows_covers_everything():
    sys.path.insert(0, str(ROOT))
    import __graft_entry__  # noqa: F401
    from dfb_b200 import replicas

    for n in (0, 1, 7, 8):
        for world in (1, 2, 3, 8):
            got = [i for r in range(world) for i in replicas.shard_rows(n, r, world)]
            assert got == list(range(n))
    with pytest.raises(ValueError):
        replicas.shard_rows(4, 2, 2)
    assert replicas.aggregate(None, 7, 1.5) == (7, 1.5)
