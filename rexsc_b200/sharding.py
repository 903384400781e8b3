"""Host-side helpers for running the hot path on several GPUs of one node.

The path shards by sample: every op is independent per batch item, weights and stream tables are replicated, so
ranks exchange nothing on the data path.  What a data-parallel caller still needs from the host side:
which slice of a global batch a rank owns, decorrelated noise seeds, a max-over-ranks reduction of timings, and a
way to keep the per-layer calibration coefficients (bias_coef / std_coef, refitted on calibration steps by the
front end, utils_functional.py:1290-1301) identical on all ranks.  Works with any torch.distributed backend
(NCCL on GPUs, gloo on CPU)."""
from __future__ import annotations

from typing import Iterable, Tuple

import torch
import torch.distributed as dist


def shard_range(global_batch: int, world: int, rank: int) -> Tuple[int, int]:
    """(start, count) of the contiguous slice of a global batch owned by `rank`; slices differ by at most one
    sample and cover the batch exactly once."""
    if world < 1 or not (0 <= rank < world) or global_batch < 0:
        raise ValueError("shard_range: need world >= 1, 0 <= rank < world, global_batch >= 0")
    base, extra = divmod(global_batch, world)
    start = rank * base + min(rank, extra)
    return start, base + (1 if rank < extra else 0)


def rank_seed(seed: int, rank: int) -> int:
    """64-bit noise seed for a rank: low word = user seed, high word = rank (see ops.manual_seed)."""
    return (int(seed) & 0xFFFFFFFF) | ((int(rank) & 0xFFFFFFFF) << 32)


def _world() -> int:
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def max_over_ranks(value: float, device=None) -> float:
    """Maximum of a per-rank scalar (e.g. a CUDA-event time in ms) over all ranks."""
    if _world() == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sync_calibration_(tensors: Iterable[torch.Tensor]) -> None:
    """Average calibration coefficient tensors in place over all ranks, so that replicas which fitted them on
    different half-batches inject the same bias / std polynomial afterwards."""
    w = _world()
    if w == 1:
        return
    for t in tensors:
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        t.div_(w)


CALIB_SUMS = 90  # 30 windows x (count, sum err, sum err^2) in the 91-entry float64 block of ops.sc_calib_stats


def reduce_calib_max_(stats: torch.Tensor) -> None:
    """All-reduce (MAX), in place, the largest count held as int32 in the first 4 bytes of entry 90 of a calibration
    block.  Called between the two stages of the statistics pass: the windows every rank then fills are those of
    the global batch.  The only exchange of the calibration path besides :func:`reduce_calib_sums_`."""
    if _world() == 1:
        return
    m = stats[CALIB_SUMS:].view(torch.int32)[:1]
    dist.all_reduce(m, op=dist.ReduceOp.MAX)


def reduce_calib_sums_(stats: torch.Tensor) -> None:
    """All-reduce (SUM), in place, the 90 window sums of a calibration block.  Valid only if every rank filled the
    same windows (see :func:`reduce_calib_max_`); afterwards every rank holds the statistics of the global batch and
    fits identical coefficients."""
    if _world() == 1:
        return
    dist.all_reduce(stats[:CALIB_SUMS], op=dist.ReduceOp.SUM)
