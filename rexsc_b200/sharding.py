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


class GradAllReducer:
    """Bucketed all-reduce (mean) of a model's weight gradients, overlapped with the rest of backward.

    This is the ONE collective a data-parallel training step of the SC models needs; the forward ops exchange
    nothing.  The reference's training loop (utils_own.py:60-198) reads ``model.fc.weight`` and writes
    ``model.sync`` on the object it is given, so the model cannot sit inside a wrapper module; instead this class
    hooks the parameters of the bare module:

    * parameters are grouped, in reverse registration order (roughly the order their gradients become ready), into
      buckets of about ``bucket_bytes``;
    * a post-accumulate-grad hook counts a bucket's gradients in; when the last one is there the bucket is flattened
      into its persistent buffer and all-reduced asynchronously (NCCL: on its own stream, over NVLink);
    * a callback queued on the autograd engine runs when backward ends: it launches buckets that never filled
      (parameters without a gradient contribute zeros, identically on every rank), waits for all reductions, divides
      by the world size and copies the means back into ``.grad``.

    With gradient accumulation (the reference steps the optimizer only after ``acc_limit`` samples) every backward
    reduces the accumulated ``.grad``; earlier contributions are already identical on all ranks, so averaging them
    again leaves them unchanged.  A GradScaler sees reduced gradients, so its inf check agrees on all ranks.
    Does nothing in a single-process job."""

    def __init__(self, module: torch.nn.Module, bucket_bytes: int = 25 << 20, process_group=None):
        self.group = process_group
        self.world = _world()
        self.params = [p for p in module.parameters() if p.requires_grad]
        self.buckets = []           # dicts: params, flat, views, pending, work
        self._bucket_of = {}
        self._queued = False
        self._handles = []
        cur, cur_bytes, cur_key = [], 0, None
        for p in reversed(self.params):
            key = (p.dtype, p.device)
            nbytes = p.numel() * p.element_size()
            if cur and (key != cur_key or cur_bytes + nbytes > bucket_bytes):
                self._add_bucket(cur)
                cur, cur_bytes = [], 0
            cur.append(p)
            cur_bytes += nbytes
            cur_key = key
        if cur:
            self._add_bucket(cur)
        if self.world > 1:
            for p in self.params:
                self._handles.append(p.register_post_accumulate_grad_hook(self._on_grad))

    # -- construction -------------------------------------------------------------------------------------------
    def _add_bucket(self, params) -> None:
        n = sum(p.numel() for p in params)
        flat = torch.zeros(n, dtype=params[0].dtype, device=params[0].device)
        views, off = [], 0
        for p in params:
            views.append(flat[off:off + p.numel()].view_as(p))
            off += p.numel()
        b = {"params": params, "flat": flat, "views": views, "pending": len(params), "work": None}
        for p in params:
            self._bucket_of[p] = b
        self.buckets.append(b)

    @property
    def nbytes(self) -> int:
        """Bytes all-reduced per backward pass."""
        return sum(b["flat"].numel() * b["flat"].element_size() for b in self.buckets)

    def remove(self) -> None:
        for h in self._handles:
            h.remove()
        self._handles = []

    # -- per backward -------------------------------------------------------------------------------------------
    def _on_grad(self, p: torch.Tensor) -> None:
        if not self._queued:
            self._queued = True
            torch.autograd.Variable._execution_engine.queue_callback(self._finish)
        b = self._bucket_of[p]
        b["pending"] -= 1
        if b["pending"] == 0:
            self._launch(b)

    def _launch(self, b) -> None:
        with torch.no_grad():
            have = [(v, p.grad) for v, p in zip(b["views"], b["params"]) if p.grad is not None]
            if len(have) != len(b["params"]):
                b["flat"].zero_()
            if have:
                torch._foreach_copy_([v for v, _ in have], [g for _, g in have])
        b["work"] = dist.all_reduce(b["flat"], op=dist.ReduceOp.SUM, group=self.group, async_op=True)

    def _finish(self) -> None:
        try:
            for b in self.buckets:
                if b["work"] is None:
                    self._launch(b)
            with torch.no_grad():
                for b in self.buckets:
                    b["work"].wait()
                    b["flat"].div_(self.world)
                    have = [(p.grad, v) for v, p in zip(b["views"], b["params"]) if p.grad is not None]
                    if have:
                        torch._foreach_copy_([g for g, _ in have], [v for _, v in have])
        finally:
            for b in self.buckets:
                b["pending"] = len(b["params"])
                b["work"] = None
            self._queued = False

    def reduce_now(self) -> None:
        """All-reduce the current ``.grad`` tensors outside of backward (used to time the collective alone)."""
        if self.world == 1:
            return
        self._finish()
