"""Synthetic-data training steps of the reference's SC models, driven through the reference's OWN training loop.

Nothing of the reference is re-implemented here: the models are built by its constructors
(``resnet_sc.resnet18/34``, resnet_sc.py:342-365; ``network.VGG16_add_partial`` / ``CONV_tiny_add_partial``,
network.py:32-125,215-272), the loss is its ``LabelSmoothLoss`` (utils.py:221-233) and every iteration runs inside
its ``utils_own.train`` (utils_own.py:201-208 -> ``forward`` :60-198: device copy, channels_last, autocast,
``loss.backward(retain_graph=True)``, GradScaler / optimizer step once ``acc_limit`` samples are in, per-iteration
scheduler step).  This module supplies what the reference gets from its datasets and command line:

* a loader of synthetic batches with the shapes and value distributions of CIFAR-10 / ImageNet-2012 inputs (the
  data sets themselves are not used), which also brackets the timed iterations with CUDA events;
* the ``sync`` mode of the step: 1 = SC bit-stream forward in every SC layer, 2 = calibration step (SC forward +
  polynomial fit, half batch as utils_own.py:117-123 does), 3 = calibrated step with error injection (no SC kernel);
* for several GPUs: one process per GPU, the batch sharded by rank, weight gradients all-reduced by
  :class:`rexsc_b200.sharding.GradAllReducer` and the calibration coefficients averaged after a ``sync=2`` step.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from .. import sharding

IMAGENET_MEAN = (0.485, 0.456, 0.406)   # normalisation constants of main_imagenet.py:139-140
IMAGENET_STD = (0.229, 0.224, 0.225)


@dataclass
class Workload:
    """One training configuration: model constructor arguments and input shape."""
    name: str
    model: str                       # resnet18 | resnet34 | vgg16 | tinyconv
    sc_compute: str
    err: object                      # int (ResNets) or list of per-stage exponents
    batch: int
    resolution: int
    classes: int
    dtype: str                       # argument of utils_own.train: fp16 | tf32 | fp32
    channels_last: bool
    generator: str = "lfsr"
    inputs: str = "imagenet"         # imagenet: clip(N(0,1),-3,3) normalised; cifar: U[0,1)
    optimizer: str = "sgd"
    acc_limit: int = 128             # samples accumulated before an optimizer step (the reference's default)
    extra: Dict = field(default_factory=dict)


WORKLOADS = {
    # SC ResNet-18, 224x224, channels_last, OR-2, 32-bit streams, fp16 autocast + GradScaler, batch 256 per GPU
    "resnet18_or2_L32": Workload("resnet18_or2_L32", "resnet18", "or_2", 5, 256, 224, 1000, "fp16", True),
    # SC ResNet-34, OR-3, 64-bit streams, batch 192 per GPU
    "resnet34_or3_L64": Workload("resnet34_or3_L64", "resnet34", "or_3", 6, 192, 224, 1000, "fp16", True),
    # VGG-16 (CIFAR shape), OR-1, 32-bit streams (128 in the classifier), NCHW, batch 256 per GPU
    "vgg16_or1_L32": Workload("vgg16_or1_L32", "vgg16", "or_1", [5, 5, 5, 5, 5, 7], 256, 32, 10, "tf32", False,
                              inputs="cifar"),
    # TinyConv on the fixed-point conv (setup c055ffbba24), batch 256
    "tinyconv_fxp": Workload("tinyconv_fxp", "tinyconv", "full_bin", [5, 5, 5, 7], 256, 32, 10, "tf32", False,
                             generator="fixed", inputs="cifar"),
}


def build_model(fe, wl: Workload, device) -> torch.nn.Module:
    """The reference's model for a workload, random initial weights (no download), on ``device``."""
    if wl.model in ("resnet18", "resnet34"):
        ctor = getattr(fe.resnet_sc, wl.model)
        model = ctor(pretrained=False, sc_compute=wl.sc_compute, uniform=False, prec=7, err=wl.err,
                     num_classes=wl.classes)
    elif wl.model == "vgg16":
        model = fe.network.VGG16_add_partial(sc_compute=wl.sc_compute, generator=wl.generator, err=wl.err)
    elif wl.model == "tinyconv":
        model = fe.network.CONV_tiny_add_partial(sc_compute=wl.sc_compute, generator=wl.generator, err=wl.err)
    else:
        raise ValueError(f"unknown model {wl.model}")
    model = model.to(device)
    if wl.channels_last:
        model = model.to(memory_format=torch.channels_last)   # main_imagenet.py:162-163
    return model


def synthetic_batch(wl: Workload, batch: int, seed: int, pinned: bool = True):
    """(inputs, labels) on the host with the distribution the workload's data set would have after the reference's
    transforms: ImageNet -> clip(N(0,1), -3, 3) then per-channel normalisation; CIFAR -> U[0,1)."""
    g = torch.Generator().manual_seed(seed)
    shape = (batch, 3, wl.resolution, wl.resolution)
    if wl.inputs == "imagenet":
        x = torch.randn(shape, generator=g).clamp_(-3, 3)
        mean = torch.tensor(IMAGENET_MEAN).view(1, 3, 1, 1)
        std = torch.tensor(IMAGENET_STD).view(1, 3, 1, 1)
        x = (x - mean) / std
    else:
        x = torch.rand(shape, generator=g)
    y = torch.randint(0, wl.classes, (batch,), generator=g)
    if pinned and torch.cuda.is_available():
        x, y = x.pin_memory(), y.pin_memory()
    return x, y


class TimedLoader:
    """Iterable standing in for a DataLoader: yields the same host batch ``warmup + steps`` times and records a CUDA
    event when the first timed iteration asks for its data and another when the last one has finished.  On a CPU
    device it falls back to wall-clock time."""

    def __init__(self, batch, warmup: int, steps: int, device, barrier: bool = False):
        self.batch, self.warmup, self.steps = batch, int(warmup), int(steps)
        self.device = torch.device(device)
        self.barrier = barrier
        self.elapsed_ms: Optional[float] = None

    def __len__(self):
        return self.warmup + self.steps

    def _sync(self):
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        if self.barrier and dist.is_available() and dist.is_initialized():
            dist.barrier()
            if self.device.type == "cuda":
                torch.cuda.synchronize(self.device)

    def __iter__(self):
        cuda = self.device.type == "cuda"
        start = end = None
        t0 = 0.0
        for i in range(self.warmup + self.steps):
            if i == self.warmup:
                self._sync()
                if cuda:
                    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    start.record(torch.cuda.current_stream(self.device))
                t0 = time.perf_counter()
            yield self.batch
        if cuda and start is not None:
            end.record(torch.cuda.current_stream(self.device))
        self._sync()
        if cuda and start is not None:
            self.elapsed_ms = start.elapsed_time(end)
        else:
            self.elapsed_ms = (time.perf_counter() - t0) * 1e3


def make_optimizer(wl: Workload, model, lr: float = 1e-3):
    """SGD with the momentum of main_conv.py:232-233 (what the metric names), or Adam as main_imagenet.py:212-213."""
    if wl.optimizer == "adam":
        return torch.optim.Adam(model.parameters(), lr=lr, weight_decay=1e-4)
    return torch.optim.SGD(model.parameters(), lr=lr, weight_decay=0, momentum=0.01)


def sc_layers(fe, model) -> List[torch.nn.Module]:
    return [m for m in model.modules() if isinstance(m, fe.utils_class.Conv2d_Add_Partial)]


class Trainer:
    """A model, optimizer, scaler and gradient all-reducer for one workload on one device (= one rank)."""

    def __init__(self, fe, wl: Workload, device, seed: int = 0, rank: int = 0, lr: float = 1e-3):
        self.fe, self.wl, self.device, self.rank = fe, wl, torch.device(device), rank
        torch.manual_seed(seed)                      # same initial weights on every rank
        self.model = build_model(fe, wl, self.device)
        self.criterion = fe.utils.LabelSmoothLoss(0.1)
        self.optimizer = make_optimizer(wl, self.model, lr)
        self.scaler = None
        if wl.dtype == "fp16":
            self.scaler = torch.amp.GradScaler("cuda" if self.device.type == "cuda" else "cpu")
        if wl.dtype == "tf32":
            torch.backends.cuda.matmul.allow_tf32 = True
            torch.backends.cudnn.allow_tf32 = True
        self.reducer = sharding.GradAllReducer(self.model)
        self.seed = seed

    def run(self, sync: int, warmup: int, steps: int, barrier: bool = True) -> Dict:
        """``warmup + steps`` iterations of utils_own.train at one ``sync`` mode; returns device time of the
        ``steps`` timed ones and the images they processed on this rank."""
        wl = self.wl
        batch = wl.batch // 2 if sync == 2 else wl.batch      # calibration steps use half a batch
        x, y = synthetic_batch(wl, batch, self.seed + 1000 * self.rank + sync)
        loader = TimedLoader((x, y), warmup, steps, self.device, barrier=barrier)
        self.model.sync = sync
        # calibrate=False: the loop then leaves model.sync alone (it would alternate 2 / 3 by iteration index);
        # acc_limit: 128 by default as in the reference, i.e. one optimizer step per iteration at these batch sizes
        self.fe.utils_own.train(loader, self.model, self.criterion, 0, self.optimizer, scaler=self.scaler,
                                dtype=wl.dtype, scheduler=None, acc_limit=wl.acc_limit,
                                channels_last=wl.channels_last, calibrate=False)
        if sync == 2:
            self.sync_calibration()
        return {"ms": loader.elapsed_ms, "images": batch * steps, "steps": steps, "batch": batch}

    def sync_calibration(self) -> None:
        """Average the layers' fitted bias / std coefficients over the ranks (each fitted its own half batch)."""
        tensors = []
        for m in sc_layers(self.fe, self.model):
            tensors += [m.bias_coef, m.std_coef]
        sharding.sync_calibration_(tensors)

    def time_allreduce(self, iters: int = 5) -> Optional[float]:
        """Device time (ms) of one bucketed all-reduce of all weight gradients, issued alone."""
        if self.reducer.world == 1 or self.device.type != "cuda":
            return None
        for p in self.reducer.params:
            if p.grad is None:
                p.grad = torch.zeros_like(p)
        self.reducer.reduce_now()
        torch.cuda.synchronize(self.device)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(iters):
            self.reducer.reduce_now()
        e.record()
        torch.cuda.synchronize(self.device)
        return s.elapsed_time(e) / iters


def blended_rate(r1: Dict, r2: Dict, r3: Dict, iters_per_epoch: int) -> float:
    """img/s of a calibrated epoch under the reference's schedule (utils_own.py:117-125): iteration ``i`` is a
    ``sync=2`` half-batch step when ``i % max(len // 5, 100) == 99`` and a ``sync=3`` step otherwise."""
    period = max(iters_per_epoch // 5, 100)
    n2 = len([i for i in range(iters_per_epoch) if i % period == 99])
    n3 = iters_per_epoch - n2
    t = n2 * r2["ms"] / r2["steps"] + n3 * r3["ms"] / r3["steps"]
    imgs = n2 * r2["batch"] + n3 * r3["batch"]
    return imgs / (t * 1e-3)


def train_block(wl_name="resnet18_or2_L32", warmup: int = 10, steps: int = 30, device=None, rank: int = 0,
                world: int = 1, modes=(3, 2, 1), fe=None) -> Dict:
    """Measure the training step of a workload per ``sync`` mode; returns the ``train`` object of the bench line
    (whole-job img/s = images of all ranks / max-over-ranks device time)."""
    from . import load

    fe = fe or load()
    wl = wl_name if isinstance(wl_name, Workload) else WORKLOADS[wl_name]
    device = torch.device(device if device is not None else ("cuda" if torch.cuda.is_available() else "cpu"))
    tr = Trainer(fe, wl, device, seed=0, rank=rank)
    out: Dict = {
        "workload": wl.name, "loop": "utils_own.train (reference, unchanged)", "optimizer": wl.optimizer,
        "autocast": wl.dtype, "batch_per_gpu": wl.batch, "warmup": warmup, "steps": steps, "n_gpus": world,
        "grad_allreduce_bytes": tr.reducer.nbytes if world > 1 else 0,
        "frontend": "byte-compiled" if fe.sourceless else "checkout",
    }
    res = {}
    for sync in modes:
        w = warmup if sync != 2 else max(3, warmup // 3)      # calibration steps are rare; keep their leg short
        k = steps if sync != 2 else max(5, steps // 3)
        r = tr.run(sync, w, k)
        r["ms"] = sharding.max_over_ranks(r["ms"], device=device if device.type == "cuda" else None)
        res[sync] = r
        out[f"sync{sync}_img_per_s"] = round(world * r["images"] / (r["ms"] * 1e-3), 1)
        out[f"sync{sync}_ms_per_step"] = round(r["ms"] / r["steps"], 3)
    if all(s in res for s in (1, 2, 3)):
        # ImageNet-2012 at this global batch: 1 281 167 images per epoch
        iters = 1281167 // (wl.batch * world) if wl.inputs == "imagenet" else 50000 // (wl.batch * world)
        out["blended_img_per_s"] = round(world * blended_rate(res[1], res[2], res[3], iters), 1)
        out["blended_schedule"] = f"{iters} iterations/epoch, sync=2 when i % max(len//5,100) == 99, else sync=3"
    ar = tr.time_allreduce()
    if ar is not None:
        out["allreduce_ms"] = round(sharding.max_over_ranks(ar, device=device), 3)
    return out
