"""world_size-2 tests of the host-side multi-GPU logic on CPU ranks (gloo): batch sharding, rank seeds,
max-over-ranks timing and calibration-coefficient averaging.  No GPU involved."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from rexsc_b200 import sharding


def test_shard_range_covers_batch_once():
    for gb in (0, 1, 7, 256, 257, 1000):
        for world in (1, 2, 3, 8):
            seen = []
            for r in range(world):
                s, c = sharding.shard_range(gb, world, r)
                seen += list(range(s, s + c))
            assert seen == list(range(gb))
            counts = [sharding.shard_range(gb, world, r)[1] for r in range(world)]
            assert max(counts) - min(counts) <= 1
    with pytest.raises(ValueError):
        sharding.shard_range(8, 2, 2)


def test_rank_seeds_are_distinct():
    seeds = {sharding.rank_seed(1234, r) for r in range(8)}
    assert len(seeds) == 8 and all(s & 0xFFFFFFFF == 1234 for s in seeds)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # each rank "measures" a different time; everyone must agree on the maximum
        t = sharding.max_over_ranks(10.0 + rank)
        # calibration coefficients fitted on different half-batches
        bias = torch.full((6,), float(rank + 1))
        std = torch.arange(6, dtype=torch.float32) * (rank + 1)
        sharding.sync_calibration_([bias, std])
        # shards of a global batch reassemble to the whole
        gb = 11
        s, c = sharding.shard_range(gb, world, rank)
        mine = torch.zeros(gb)
        mine[s:s + c] = 1
        dist.all_reduce(mine)
        out.put((rank, t, bias.tolist(), std.tolist(), mine.tolist()))
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, t, bias, std, mine in results:
        assert t == 11.0
        assert bias == [1.5] * 6
        assert std == [1.5 * i for i in range(6)]
        assert mine == [1.0] * 11
