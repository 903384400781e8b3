"""world_size-2 tests of the host-side multi-GPU logic on CPU ranks (gloo): batch sharding, rank seeds,
max-over-ranks timing, calibration-coefficient averaging and calibration over a batch sharded across ranks (maximum
and window sums all-reduced, identical fit on every rank).  No GPU involved: the device pass that fills a rank's
statistics block is stood in for by the oracle."""
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


def _calib_shard(rank, world, n=6000, L=32):
    g = torch.Generator().manual_seed(11)
    act = torch.rand(2 * n, generator=g) ** 2 * 1.9
    cnt = torch.round((act * (1 - 0.04 * act) + 0.04 * torch.randn(2 * n, generator=g)) * L).clamp(0, 2 * L)
    cnt[0] = 2 * L  # the global maximum lives in rank 0's shard only
    s, c = sharding.shard_range(2 * n, world, rank)
    return act, cnt, slice(s, s + c), L


def _calib_worker(rank, world, port, out):
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle"))
    import oracle
    from rexsc_b200 import ops

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        act, cnt, mine, L = _calib_shard(rank, world)
        block = torch.zeros(91, dtype=torch.float64)
        block[90:].view(torch.int32)[0] = int(cnt[mine].max())          # what rexsc_sc_calib_max leaves
        sharding.reduce_calib_max_(block)
        top = int(block[90:].view(torch.int32)[0]) / L
        sums = oracle.calib_window_sums(cnt[mine].numpy() / L, act[mine].numpy(), top)  # rexsc_sc_calib_windows
        block[:90] = torch.from_numpy(sums.reshape(-1))
        sharding.reduce_calib_sums_(block)
        bias, std = ops.fit_bias_std_coef(block, L, 5)
        out.put((rank, int(block[90:].view(torch.int32)[0]), block[:90].tolist(), bias.tolist(), std.tolist()))
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_calibrate_on_the_global_batch(oracle):
    import numpy as np

    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_calib_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=180) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    act, cnt, _, L = _calib_shard(0, 1)
    whole = oracle.calib_window_sums(cnt.numpy() / L, act.numpy())
    ref_bias, ref_std = oracle.compute_bias_std_coef(2, cnt / L, act, 5)
    starts = np.linspace(0, float(cnt.max()) / L, 30)
    assert results[0][1:3] == results[1][1:3]                    # both ranks hold the same block, bit for bit
    for a, b in zip(results[0][3:], results[1][3:]):             # and fit the same polynomials (CPU LAPACK: to 1e-4)
        assert np.allclose(a, b, rtol=1e-4, atol=1e-6)
    for _, max_count, sums, bias, std in results:
        assert max_count == int(cnt.max())
        assert np.allclose(np.array(sums).reshape(30, 3), whole, rtol=1e-12, atol=1e-9)
        for ours, ref in ((bias, ref_bias), (std, ref_std)):
            pa = sum(c * starts ** i for i, c in enumerate(ours))
            pr = sum(float(c) * starts ** i for i, c in enumerate(ref))
            assert np.allclose(pa, pr, atol=1e-4)
