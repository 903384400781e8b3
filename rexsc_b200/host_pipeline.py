"""SC conv forward for callers whose tensors live in HOST memory.

``HostConvPipeline.run`` takes a list of conv calls whose activations are pinned host tensors and whose results
are wanted in pinned host tensors, and overlaps the three phases of consecutive calls on three CUDA streams:
host->device copy of call i+1, compute of call i, device->host copy of call i-1.  Device staging buffers are
double-buffered per tensor shape.  Results are identical to calling ``ops.conv2d_generic_general_split_acc`` on
device copies; only the schedule differs.  With ``chunks > 1`` every call is run as that many calls on consecutive
slices of the batch (images are independent in the SC conv: seeds depend on channel and position only), which
shortens the ramp at both ends of a run: the first copy-in and the last copy-out are a chunk long, not a batch long.
"""
from __future__ import annotations

from typing import Dict, List, Sequence

import torch

from . import ops


class HostConvCall:
    """One SC conv2d forward: pinned host activation in, pinned host int16 outputs out; the weight stays on the
    device (weights change once per optimizer step, activations every call)."""

    def __init__(self, x_host: torch.Tensor, weight_dev: torch.Tensor, out_pos_host: torch.Tensor,
                 out_neg_host: torch.Tensor, bit_length: int, stride: Sequence[int], bin_config: int,
                 padding: Sequence[int] = (0, 0), lfsr_length: int = -1, prog_load: Sequence[int] = (7, 8, 1),
                 gen_config: int = 1, xnor: bool = True):
        self.x_host, self.weight_dev = x_host, weight_dev
        self.out_pos_host, self.out_neg_host = out_pos_host, out_neg_host
        self.args = (bit_length, lfsr_length, 16, tuple(padding), tuple(stride), tuple(prog_load), bin_config,
                     gen_config, xnor, False)

    def narrow(self, start: int, length: int) -> "HostConvCall":
        """The same call on images [start, start + length) of the batch (views of the same host tensors)."""
        sub = HostConvCall.__new__(HostConvCall)
        sub.x_host = self.x_host.narrow(0, start, length)
        sub.weight_dev = self.weight_dev
        sub.out_pos_host = self.out_pos_host.narrow(0, start, length)
        sub.out_neg_host = self.out_neg_host.narrow(0, start, length)
        sub.args = self.args
        return sub


class HostConvPipeline:
    def __init__(self, device, slots: int = 2, chunks: int = 1):
        self.device = torch.device(device)
        self.slots = slots
        self.chunks = max(1, int(chunks))
        self.s_in = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)
        self._stage: Dict[tuple, List[torch.Tensor]] = {}

    def _buffers(self, kind: str, like: torch.Tensor) -> List[torch.Tensor]:
        key = (kind, tuple(like.shape), like.dtype, tuple(like.stride()))
        bufs = self._stage.get(key)
        if bufs is None:
            bufs = [torch.empty_strided(like.shape, like.stride(), dtype=like.dtype, device=self.device)
                    for _ in range(self.slots)]
            self._stage[key] = bufs
        return bufs

    def run(self, calls: Sequence[HostConvCall]) -> None:
        """Enqueue all calls; returns after everything is enqueued.  Synchronise the device (or the current
        stream plus ``self.s_out``) before reading the host outputs."""
        dev = self.device
        compute = torch.cuda.current_stream(dev)
        # per (kind, shape) ring position and the events that say when a staging buffer may be reused
        ring: Dict[tuple, int] = {}
        free_after: Dict[int, torch.cuda.Event] = {}
        self.s_in.wait_stream(compute)
        self.s_out.wait_stream(compute)
        if self.chunks > 1:
            split = []
            for c in calls:
                n = c.x_host.size(0)
                k = min(self.chunks, n)
                bounds = [n * i // k for i in range(k + 1)]
                split.extend(c.narrow(bounds[i], bounds[i + 1] - bounds[i]) for i in range(k))
            calls = split
        for c in calls:
            xb = self._buffers("x", c.x_host)
            pb = self._buffers("p", c.out_pos_host)
            nb = self._buffers("n", c.out_neg_host)
            kx = ("x", id(xb))
            ko = ("o", id(pb))
            ix = ring.get(kx, 0)
            io = ring.get(ko, 0)
            ring[kx] = (ix + 1) % self.slots
            ring[ko] = (io + 1) % self.slots
            x_dev, p_dev, n_dev = xb[ix], pb[io], nb[io]
            # 1. host -> device, once the previous user of this input buffer has finished computing
            ev = free_after.get(id(x_dev))
            if ev is not None:
                self.s_in.wait_event(ev)
            with torch.cuda.stream(self.s_in):
                x_dev.copy_(c.x_host, non_blocking=True)
                ev_in = torch.cuda.Event()
                ev_in.record(self.s_in)
            # 2. compute, once the input has landed and the previous user of the output buffers was copied out
            compute.wait_event(ev_in)
            ev = free_after.get(id(p_dev))
            if ev is not None:
                compute.wait_event(ev)
            ops.conv2d_generic_general_split_acc(x_dev, c.weight_dev, *c.args, out=(p_dev, n_dev))
            ev_comp = torch.cuda.Event()
            ev_comp.record(compute)
            free_after[id(x_dev)] = ev_comp
            # 3. device -> host
            self.s_out.wait_event(ev_comp)
            with torch.cuda.stream(self.s_out):
                c.out_pos_host.copy_(p_dev, non_blocking=True)
                c.out_neg_host.copy_(n_dev, non_blocking=True)
                ev_out = torch.cuda.Event()
                ev_out.record(self.s_out)
            free_after[id(p_dev)] = ev_out
        compute.wait_stream(self.s_out)
