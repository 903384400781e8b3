#!/usr/bin/env python
"""Benchmark of the SC arithmetic hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config NAME]

Default workload (``--config resnet18``): the SC forward hot path of SC ResNet-18 at 224x224, channels_last, OR-2
with 32-bit streams, batch 256 per GPU -- for each of the 19 SC conv layers one call of
conv2d_generic_general_split_acc (pad + quantise + LFSR streams + OR-n accumulation) exactly as
utils_functional.py:1179 of the reference calls it, followed by the OR-n activation of the float guide
(or_approx_n_forward_acc on the pos and the neg sum).  Synthetic inputs: activations uniform in [0,1) quantised
to 7 bits (what the reference's Hardtanh + QuantizeGrad feed the op), weights N(0, 0.1) clipped to [-1, 1].
Other workloads, same measurement: ``resnet34`` (OR-3, 64-bit streams, batch 192), ``vgg16`` (CIFAR shape, NCHW,
OR-1, batch 256), ``conv5x5`` (the single 3->32 5x5 conv), ``linear`` (SC linear 512->512->10), ``tinyconv_fxp``
(the four fixed-point conv layers of TinyConv).

One JSON line is printed by rank 0:
  value      images/s with inputs resident in HBM, CUDA-event time, max over ranks, whole job
  e2e        the same through the op-level API with HOST (pinned) buffers: H2D of every layer's activation and
             D2H of every layer's int16 outputs inside the timed region (fp16 activations, as the front end passes
             them under autocast; `e2e_fp32_activations` repeats it with fp32 activations); --e2e-slots / --e2e-chunks
             set the staging depth and the batch slicing of the host pipeline
  gpu_launches  this library's kernels inside the timed region, as the library counts them
  roofline   dominant kernel: the tensor-core SC conv (one int8 tcgen05 GEMM per time slot) against the int8 tensor
             rate measured live by a back-to-back MMA probe; `roofline_secondary` / `roofline_expand` the ALU kernel
             and the stream-expansion stage; `roofline_pointwise` the four point-wise kernels against HBM
  train      images/s of full training steps (fwd + bwd + optimizer) of the reference's own model and loop on the
             drop-in ops, per `sync` mode, with the NCCL weight-gradient all-reduce when N > 1
  cpu_baseline  the reference's own CPU extension (oracle/_ref) on a bounded sample, N=1 only
`--impl reference` times that CPU extension alone (all host threads) on the same layer list at a reduced batch.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PROG = (7, 8, 1)


# ---- workloads ------------------------------------------------------------------------------------------
# layer = (c_in, spatial size of the UNPADDED input, c_out, kernel, stride, pad, repeats, stream length)
def _resnet_layers(blocks, L):
    """SC conv layers of resnet_sc.py's BasicBlock ResNets at 224x224 (first conv and FC are float layers)."""
    out, cin, h = [], 64, 56
    for stage, (cout, n) in enumerate(zip((64, 128, 256, 512), blocks)):
        if stage == 0:
            out.append((64, 56, 64, 3, 1, 1, 2 * n, L))
            continue
        out.append((cin, h, cout, 3, 2, 1, 1, L))          # first conv of the stage, stride 2
        out.append((cin, h, cout, 1, 2, 0, 1, L))          # 1x1 shortcut
        h //= 2
        out.append((cout, h, cout, 3, 1, 1, 2 * n - 1, L))
        cin = cout
    return out


def _vgg16_layers():
    """network.py:32-125: thirteen 3x3 pad-1 SC convs on 32x32 inputs and the 1x1 classifier with 128-bit streams."""
    cfg = [(3, 32, 64), (64, 32, 64), (64, 16, 128), (128, 16, 128), (128, 8, 256), (256, 8, 256), (256, 8, 256),
           (256, 4, 512), (512, 4, 512), (512, 4, 512), (512, 2, 512), (512, 2, 512), (512, 2, 512)]
    return [(ci, h, co, 3, 1, 1, 1, 32) for ci, h, co in cfg] + [(512, 1, 10, 1, 1, 0, 1, 128)]


WORKLOADS = {
    "resnet18": dict(
        kind="sc", metric="sc_resnet18_or2_L32_sc_forward_img_per_s", batch=256, or_n=2, channels_last=True,
        layers=_resnet_layers((2, 2, 2, 2), 32), guide_dtype=torch.float16,
        text="SC ResNet-18 224x224 channels_last OR-2 L=32 batch 256/GPU: 19 SC conv2d forwards (padded activations "
             "in, int16 pos/neg out) + 38 OR-n activation forwards (fp16 in)"),
    "resnet34": dict(
        kind="sc", metric="sc_resnet34_or3_L64_sc_forward_img_per_s", batch=192, or_n=3, channels_last=True,
        layers=_resnet_layers((3, 4, 6, 3), 64), guide_dtype=torch.float16,
        text="SC ResNet-34 224x224 channels_last OR-3 L=64 batch 192/GPU: 35 SC conv2d forwards + 70 OR-n activation "
             "forwards (fp16 in)"),
    "vgg16": dict(
        kind="sc", metric="sc_vgg16_or1_L32_sc_forward_img_per_s", batch=256, or_n=1, channels_last=False,
        layers=_vgg16_layers(), guide_dtype=torch.float32,
        text="SC VGG-16 (CIFAR shape) NCHW OR-1 L=32 (classifier L=128) batch 256/GPU: 14 SC conv2d forwards + 28 OR-n "
             "activation forwards (fp32 in)"),
    "conv5x5": dict(
        kind="sc", metric="sc_conv5x5_or1_L32_forward_img_per_s", batch=32, or_n=1, channels_last=False,
        layers=[(3, 32, 32, 5, 1, 2, 1, 32)], guide_dtype=torch.float32,
        text="one SC conv2d forward, N=32, 3->32 channels, 5x5, pad 2, 32x32, OR-1 L=32, NCHW + 2 OR-n activation "
             "forwards"),
    "linear": dict(
        kind="linear", metric="sc_linear_512_512_10_or1_L128_rows_per_s", batch=256, or_n=1,
        layers=[(512, 512, 128), (512, 10, 128)],
        text="SC linear 512->512->10 (linear_generic_general_acc), OR-1, 128-bit streams, 256 rows per step"),
    "tinyconv_fxp": dict(
        kind="fxp", metric="fxp_tinyconv_forward_img_per_s", batch=256,
        # (c_in, unpadded size, c_out, kernel, pad, precision_in)
        layers=[(3, 32, 32, 5, 2, 5), (32, 16, 32, 5, 2, 5), (32, 8, 64, 5, 2, 5), (64, 4, 10, 4, 0, 7)],
        text="FXP TinyConv batch 256: four conv2d_saturate_acc forwards (3->32 @32x32, 32->32 @16x16, 32->64 @8x8, "
             "5x5 pad 2, 5-bit; 64->10 4x4, 7-bit), 24-bit saturating accumulation"),
}
TRAIN_WORKLOAD = {"resnet18": "resnet18_or2_L32", "resnet34": "resnet34_or3_L64", "vgg16": "vgg16_or1_L32",
                  "tinyconv_fxp": "tinyconv_fxp"}


def layer_out(h, k, s, p):
    return (h + 2 * p - k) // s + 1


def products_per_image(layers):
    return sum(rep * layer_out(h, k, s, p) ** 2 * cout * cin * k * k for cin, h, cout, k, s, p, rep, L in layers)


def bitops_per_image(layers):
    """2 * L * OH*OW * Cout * Cin*KH*KW summed over the SC layers (pos and neg streams, useful channels)."""
    return sum(rep * 2 * L * layer_out(h, k, s, p) ** 2 * cout * cin * k * k for cin, h, cout, k, s, p, rep, L in layers)


# ------------------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-i", str(self.gpu),
                 "-lms", "25"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, mx, reasons = [], None, set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 8:
                continue
            try:
                clocks.append(float(f[1]))
                mx = float(f[2])
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        busy = sorted(c for c in clocks if mx is None or c > 0.5 * mx) or sorted(clocks)
        med = busy[len(busy) // 2] if busy else None
        return {"sm_mhz": med, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(clocks)}


def _hbm_peak():
    try:
        return float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"])
    except Exception:
        return 6650.0


def _hbm_peak_source():
    return "MEASURED_PEAKS.json (of measured)" if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) \
        else "6.65 TB/s (of fallback)"


def _event_ms(fn, reps=5, warm=2):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / reps


def _timed_steps(step_fn, steps, warmup, world, dev, sharding):
    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        step_fn()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step_fn()
    e1.record()
    barrier()
    return sharding.max_over_ranks(e0.elapsed_time(e1), device=dev)


def _mma_peak(ops, dev):
    """int8 ops / s of back-to-back tcgen05 MMAs on fixed operands (2 per multiply-accumulate)."""
    ops.mma_probe(296, 100, 128, dev)
    t = min(_event_ms(lambda: ops.mma_probe(296, 4000, 128, dev), reps=1, warm=0) for _ in range(3))
    return 2.0 * 296 * 4000 * 16 * 128 * 128 * 32 / (t * 1e-3)


def make_layers(wl, batch, seed):
    """Per distinct layer shape: padded activation and weight in the workload's memory format, stride."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    fmt = torch.channels_last if wl["channels_last"] else torch.contiguous_format
    layers = []
    for cin, h, cout, k, s, p, rep, L in wl["layers"]:
        x = torch.rand(batch, cin, h, h, generator=g)
        x = (x * 128).round().clamp(0, 127) / 128
        x = torch.nn.functional.pad(x, (p, p, p, p)).contiguous(memory_format=fmt)
        w = (torch.randn(cout, cin, k, k, generator=g) * 0.1).clamp(-1, 1)
        w = ((w * 128).round().clamp(-127, 127) / 128).contiguous(memory_format=fmt)
        layers.append({"x_host": x, "w_host": w, "stride": s, "rep": rep, "L": L, "shape": (cin, h, cout, k, s, p)})
    return layers


def _sc_desc(_lib, l, wl, x, w, act_dtype=0):
    d = _lib.ScConvDesc()
    d.batch, d.c_in, d.h_in, d.w_in = x.shape
    d.c_out, _, d.kh, d.kw = w.shape
    d.stride_h = d.stride_w = l["stride"]
    cl = 1 if wl["channels_last"] else 0
    d.act_dtype, d.act_channels_last, d.w_dtype, d.w_channels_last, d.out_channels_last = act_dtype, cl, 0, cl, cl
    d.bit_length, d.lfsr_length, d.bin_config, d.gen_config, d.xnor = l["L"], -1, wl["or_n"] - 1, 1, 1
    d.prog_total_width, d.prog_load_width, d.prog_load_wait = PROG
    return d


# ---- SC conv workloads -------------------------------------------------------------------------------------
def run_sc(args, wl, rank, world, local_rank):
    from rexsc_b200 import _lib, ops, sharding
    from rexsc_b200.host_pipeline import HostConvCall, HostConvPipeline

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    lib = _lib.load()  # fails loudly if the CUDA library is missing
    batch, or_n = wl["batch"], wl["or_n"]
    fmt = torch.channels_last if wl["channels_last"] else torch.contiguous_format
    layers = make_layers(wl, batch, seed=1000 + rank)
    for l in layers:
        l["x"] = l["x_host"].to(dev).contiguous(memory_format=fmt)
        l["w"] = l["w_host"].to(dev).contiguous(memory_format=fmt)
        l["x_pin16"] = l["x_host"].half().contiguous(memory_format=fmt).pin_memory()
        l["x_pin32"] = l["x_host"].pin_memory()
    def conv(l, x):
        return ops.conv2d_generic_general_split_acc(x, l["w"], l["L"], -1, 16, (0, 0), (l["stride"],) * 2, PROG,
                                                    or_n - 1, 1, True, False)

    # float guide sums for the point-wise kernels: synthetic conv sums of the right shape (dtype as the front end has)
    guides = {}
    for i, l in enumerate(layers):
        # kernels per conv call, counted by the library: the single-launch expand stage and the tensor-core kernel,
        # plus -- for 3x3 stride-1 layers, whose padding the caller did -- the gated fallback pair and the clearing of
        # the tiles that CTAs share; four or more on the ALU paths (tables, two expansions, accumulate)
        c0 = lib.rexsc_kernel_launch_count()
        p, n = conv(l, l["x"])
        l["kernels"] = lib.rexsc_kernel_launch_count() - c0
        g = torch.Generator(device=dev).manual_seed(7 + i)
        guides[i] = (torch.rand(p.shape, device=dev, generator=g, dtype=torch.float32).to(wl["guide_dtype"])
                     .contiguous(memory_format=fmt) * 4)

    def step_resident():
        for i, l in enumerate(layers):
            for _ in range(l["rep"]):
                conv(l, l["x"])
                ops.or_approx_n_forward_acc(guides[i], or_n)
                ops.or_approx_n_forward_acc(guides[i], or_n)

    # host-facing step: every call takes pinned host tensors and returns host tensors
    out_pin = {}
    for i, l in enumerate(layers):
        p, n = conv(l, l["x"])
        out_pin[i] = (torch.empty(p.shape, dtype=p.dtype).contiguous(memory_format=fmt).pin_memory(),
                      torch.empty(n.shape, dtype=n.dtype).contiguous(memory_format=fmt).pin_memory())
    d2h = sum(out_pin[i][0].numel() * 2 * 2 * l["rep"] for i, l in enumerate(layers))
    pipe = HostConvPipeline(dev, slots=args.e2e_slots, chunks=args.e2e_chunks)

    def host_step(key):
        calls = []
        for i, l in enumerate(layers):
            for _ in range(l["rep"]):
                calls.append(HostConvCall(l[key], l["w"], out_pin[i][0], out_pin[i][1], l["L"], (l["stride"],) * 2,
                                          or_n - 1))

        def step():
            # host buffers in, host buffers out: H2D / compute / D2H of consecutive calls overlap on three streams
            pipe.run(calls)
            for i, l in enumerate(layers):
                for _ in range(l["rep"]):
                    ops.or_approx_n_forward_acc(guides[i], or_n)
                    ops.or_approx_n_forward_acc(guides[i], or_n)
        return step, sum(l[key].numel() * l[key].element_size() * l["rep"] for l in layers)

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    c0 = lib.rexsc_kernel_launch_count()
    ms = _timed_steps(step_resident, args.steps, args.warmup, world, dev, sharding)
    # this library's kernels inside the timed region, as the library counted them (warm-up steps taken out)
    n_launch = (lib.rexsc_kernel_launch_count() - c0) * args.steps // (args.steps + args.warmup)
    clocks = sampler.stop() if rank == 0 else None
    e2e_steps = max(1, min(args.steps, 5))
    step16, h2d16 = host_step("x_pin16")
    ms_e2e16 = _timed_steps(step16, e2e_steps, 1, world, dev, sharding)
    step32, h2d32 = host_step("x_pin32")
    ms_e2e32 = _timed_steps(step32, e2e_steps, 1, world, dev, sharding)

    # per-direction copy rates of this rank with both directions busy on every rank at once (what bounds e2e)
    big_in = max((l["x_pin32"] for l in layers), key=lambda t: t.numel())
    big_out = max((out_pin[i][0] for i in out_pin), key=lambda t: t.numel())
    din, dout = torch.empty_like(big_in, device=dev), torch.empty_like(big_out, device=dev)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

    def both_ways(reps=3):
        """GB/s of each direction, measured on its own stream while the other direction is busy too."""
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        torch.cuda.synchronize()
        with torch.cuda.stream(s_in):
            ev[0].record(s_in)
            for _ in range(reps):
                din.copy_(big_in, non_blocking=True)
            ev[1].record(s_in)
        with torch.cuda.stream(s_out):
            ev[2].record(s_out)
            for _ in range(2 * reps):
                big_out.copy_(dout, non_blocking=True)
            ev[3].record(s_out)
        torch.cuda.synchronize()
        return (reps * big_in.numel() * 4 / ev[0].elapsed_time(ev[1]) / 1e6,
                2 * reps * big_out.numel() * 2 / ev[2].elapsed_time(ev[3]) / 1e6)

    if world > 1:
        torch.distributed.barrier()
    both_ways(1)
    h2d_gbs, d2h_gbs = both_ways()
    link = {"h2d_gbs": -sharding.max_over_ranks(-h2d_gbs, device=dev),    # slowest rank
            "d2h_gbs": -sharding.max_over_ranks(-d2h_gbs, device=dev)}
    del din, dout

    # ---- accumulate kernels timed alone per layer with CUDA events (same stream, after the layer's expand stage) ----
    per_kernel = {k: {"ms": 0.0, "products": 0, "launches": 0, "intops": 0.0, "lop3": 0.0, "bytes": 0, "plane_bytes": 0}
                  for k in ("tensor", "tiled", "direct")}
    per_layer = []
    exp_ms, exp_bytes = 0.0, 0
    lop3_per_product = {1: 1, 2: 3, 3: 4, 4: 5}[or_n]
    for l in layers:
        x, w = l["x"], l["w"]
        d = _sc_desc(_lib, l, wl, x, w)
        which_kernel = {1: "direct", 2: "tiled", 3: "tensor"}[lib.rexsc_sc_conv2d_kernel_choice(C.byref(d))]
        nbytes = lib.rexsc_sc_conv2d_workspace_size(C.byref(d))
        ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        oh = (d.h_in - d.kh) // d.stride_h + 1
        pos = torch.empty((d.batch, d.c_out, oh, oh), dtype=torch.int16, device=dev, memory_format=fmt)
        neg = torch.empty_like(pos)
        st = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        vp = lambda t: C.c_void_p(t.data_ptr())
        best = {}
        for which in ("expand", "accumulate"):
            for it in range(4):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                if which == "expand":
                    rc = lib.rexsc_sc_conv2d_expand(C.byref(d), vp(x), vp(w), vp(ws), nbytes, st)
                else:
                    rc = lib.rexsc_sc_conv2d_accumulate(C.byref(d), vp(pos), vp(neg), vp(ws), nbytes, st)
                e1.record()
                torch.cuda.synchronize()
                _lib.check(rc, which)
                t = e0.elapsed_time(e1)
                if it > 0:
                    best[which] = t if which not in best else min(best[which], t)
        slots = l["L"]
        px = d.batch * d.h_in * d.w_in
        plane_bytes = slots // 8 * ((d.c_in + 31) // 32 * 32) * px
        exp_ms += best["expand"] * l["rep"]
        # algorithmic bytes of the stage: the activations read once + their bit planes (or stream words) written once,
        # one bit per element and time slot, channels padded to whole 32-bit words
        exp_bytes += l["rep"] * (x.numel() * x.element_size() + plane_bytes)
        k = per_kernel[which_kernel]
        products = batch * oh * oh * d.c_out * d.c_in * d.kh * d.kw
        k["ms"] += best["accumulate"] * l["rep"]
        k["products"] += l["rep"] * products
        k["launches"] += l["rep"]
        k["intops"] += l["rep"] * 4.0 * slots * products          # int8 ops of the per-slot GEMMs
        k["lop3"] += l["rep"] * float(lop3_per_product) * products * ((slots + 31) // 32)
        # DRAM bytes the accumulate kernel has to move: the activation bit planes once + both int16 outputs
        k["bytes"] += l["rep"] * (plane_bytes + 2 * 2 * d.batch * oh * oh * d.c_out)
        k["plane_bytes"] += l["rep"] * plane_bytes
        per_layer.append({"shape": list(l["shape"]), "L": slots, "kernel": which_kernel, "rep": l["rep"],
                          "expand_ms": round(best["expand"], 4), "accumulate_ms": round(best["accumulate"], 4),
                          "tbitops_per_s": round(2 * slots * products / (best["accumulate"] * 1e-3) / 1e12, 1)})
        del ws, pos, neg

    mma_peak_ops = _mma_peak(ops, dev)
    # ---- live LOP3 peak (register-only probe) ------------------------------------------------------------
    blocks, iters = 148 * 8, 20000
    ops.alu_probe(blocks, 200, dev)
    t = min(_event_ms(lambda: ops.alu_probe(blocks, iters, dev), reps=1, warm=0) for _ in range(3))
    lop3_peak = blocks * 256 * iters * 64 / (t * 1e-3)  # lane-ops / s

    # ---- point-wise kernels on the largest layer's guide tensor (> L2 for the ImageNet workloads) ---------------
    gbig = max(guides.values(), key=lambda t: t.numel())
    n_el, bi = gbig.numel(), gbig.element_size()
    gneg = gbig.flip(0).contiguous(memory_format=fmt)
    grad = torch.randn(gbig.shape, device=dev).contiguous(memory_format=fmt)
    bias = torch.tensor([0.01, -0.05, 0.02, 0.003, -0.001, 0.0002], device=dev)
    std = torch.tensor([0.02, 0.05, -0.01, 0.002, 0.0, 0.0001], device=dev)
    dtn = "half" if bi == 2 else "float"
    pw = []
    for name, fn, nbytes in (
            (f"pw_kernel<OrnFwd<{dtn},{or_n}>>", lambda: ops.or_approx_n_forward_acc(gbig, or_n), bi + 4),
            (f"pw_kernel<OrnBwd<{dtn},{or_n}>>", lambda: ops.or_approx_n_backward_acc(grad, gbig, or_n), bi + 8),
            (f"both_fwd_kernel<{dtn},{or_n}> (fused calibration + error injection forward)",
             lambda: ops.or_approx_n_forward_bias_std_both_acc(gbig, gneg, bias, std, or_n), 2 * bi + 4),
            (f"pw_kernel<BothBwd<{dtn},{or_n}>> (fused calibration backward)",
             lambda: ops.or_approx_n_backward_bias_std_both_acc(grad, gbig, gneg, bias, or_n), 2 * bi + 12)):
        gbs = n_el * nbytes / (_event_ms(fn) * 1e-3) / 1e9
        pw.append({"bound": "hbm", "kernel": name, "achieved": gbs, "unit": "GB/s", "peak": _hbm_peak(),
                   "frac": gbs / _hbm_peak(), "bytes_per_element": nbytes, "elements": n_el,
                   "peak_source": _hbm_peak_source()})
    del gneg, grad

    # ---- caller arithmetic on the counts of the largest layer: counts -> fp16 values, calibration windows ----
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    val = [torch.rand(gbig.shape, device=dev, generator=gen).contiguous(memory_format=fmt) ** 2 * 1.9 for _ in range(2)]
    L0 = layers[0]["L"]
    cnt = [torch.round((v * (1 - 0.04 * v) + 0.05 * torch.randn(v.shape, device=dev, generator=gen).contiguous(
        memory_format=fmt)) * L0).clamp(0, or_n * L0).to(torch.int16) for v in val]
    # int16 pos + neg in, fp16 pos / neg values out (what the front end builds under autocast)
    c2v_gbs = n_el * 8 / (_event_ms(lambda: ops.sc_counts_to_value(cnt[0], cnt[1], L0, torch.float16)) * 1e-3) / 1e9
    # counts read twice (maximum, then windows) + both fp32 guide tensors once
    calib_gbs = n_el * 16 / (_event_ms(lambda: ops.sc_calib_stats(cnt[0], cnt[1], val[0], val[1], L0)) * 1e-3) / 1e9
    del val, cnt
    return {"ms": ms, "launches": n_launch, "e2e_steps": e2e_steps, "ms_e2e16": ms_e2e16, "ms_e2e32": ms_e2e32,
            "h2d16": h2d16, "h2d32": h2d32, "d2h": d2h, "link": link, "clocks": clocks, "per_kernel": per_kernel,
            "per_layer": per_layer, "exp_ms": exp_ms, "exp_bytes": exp_bytes, "lop3_peak": lop3_peak,
            "mma_peak_ops": mma_peak_ops, "pw": pw, "c2v_gbs": c2v_gbs, "calib_gbs": calib_gbs}


def sc_line(args, wl, r, world):
    batch = wl["batch"]
    value = batch * world * args.steps / (r["ms"] * 1e-3)
    e2e16 = batch * world * r["e2e_steps"] / (r["ms_e2e16"] * 1e-3)
    e2e32 = batch * world * r["e2e_steps"] / (r["ms_e2e32"] * 1e-3)
    pk = r["per_kernel"]
    t, a = pk["tensor"], pk["tiled"]
    tc_achieved = t["intops"] / (t["ms"] * 1e-3) if t["ms"] > 0 else 0.0
    alu_achieved = a["lop3"] / (a["ms"] * 1e-3) if a["ms"] > 0 else 0.0
    roof_tensor = {
        "bound": "tensor", "kernel": "sc_conv_tc_kernel (tcgen05 int8, one GEMM per time slot)",
        "achieved": tc_achieved / 1e12, "peak": r["mma_peak_ops"] / 1e12, "unit": "TOP/s int8",
        "frac": tc_achieved / r["mma_peak_ops"],
        # per average launch: reads = 1.23 x the activation bit planes, the ratio of ncu's dram__bytes_read.sum
        # (65.6 MB) to the planes (53.2 MB) of the captured 64-channel layer at batch 64 (patch halos, the
        # read-modify-write of cut tiles and the weight planes make up the rest; it grows in proportion to the batch);
        # writes = the int16 outputs (a single captured launch leaves most of them in L2 -- 13.0 of 51.4 MB had been
        # written back when the capture ended -- a whole step, whose layers do not fit L2 together, writes them all)
        "traffic": ((0.23 * t["plane_bytes"] + t["bytes"]) / t["launches"]) if t["launches"] else None,
        "traffic_source": "ncu capture of one layer at batch 64 (read ratio), scaled by algorithmic bytes",
        "peak_source": "measured live: back-to-back tcgen05.mma kind::i8 M128 N128 K32 probe on this GPU",
        "kernel_ms_per_step": t["ms"], "launches_per_step": t["launches"],
        "tbitops_per_s_kernel": t["intops"] / 2 / (t["ms"] * 1e-3) / 1e12 if t["ms"] > 0 else 0.0,
    }
    roof_alu = {
        "bound": "alu", "kernel": "sc_conv_tiled_kernel (LOP3 thermometer OR-n; thin inputs, large filters)",
        "achieved": alu_achieved / 1e12, "peak": r["lop3_peak"] / 1e12, "unit": "T lane-LOP3/s",
        "frac": alu_achieved / r["lop3_peak"], "traffic": None,
        "peak_source": "measured live: register-only LOP3 probe on this GPU (integer ALU pipe)",
        "kernel_ms_per_step": a["ms"], "launches_per_step": a["launches"],
    }
    exp_gbs = r["exp_bytes"] / (r["exp_ms"] * 1e-3) / 1e9 if r["exp_ms"] > 0 else 0.0
    roof_expand = {
        "bound": "hbm", "kernel": "expand stage (stream tables + activation and weight expansion, per layer)",
        "achieved": exp_gbs, "peak": _hbm_peak(), "unit": "GB/s", "frac": exp_gbs / _hbm_peak(), "traffic": None,
        "peak_source": _hbm_peak_source(), "kernel_ms_per_step": r["exp_ms"],
    }
    dominant, secondary = (roof_tensor, roof_alu) if t["ms"] >= a["ms"] else (roof_alu, roof_tensor)
    dominant["expand_ms_per_step"] = r["exp_ms"]
    big = batch * products_per_image(wl["layers"]) > 1e11
    line = {
        "metric": wl["metric"], "value": value, "unit": "img/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms"] / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "u32 bit-streams / int8 tensor-core operands, int32 accumulators / int16 sums", "data": "synthetic",
        "config": {
            "workload": wl["text"], "batch_per_gpu": batch,
            "parallelism": f"batch-sharded x{world}, no data-path collective on the forward ops "
                           "(the train block all-reduces weight gradients)",
            "l2_policy": "inputs larger than L2 (more than 1 GB of layer activations per step)" if big
            else "small workload: the step's working set may stay in L2, reported as such",
        },
        "tbitops_per_s": bitops_per_image(wl["layers"]) * value / 1e12,
        "e2e": {"value": e2e16, "unit": "img/s", "h2d_bytes_per_step": r["h2d16"], "d2h_bytes_per_step": r["d2h"],
                "activations": "fp16 (what the front end passes under autocast)",
                "pipeline": f"HostConvPipeline: copy-in / compute / copy-out of consecutive calls on three streams, "
                            f"{args.e2e_slots} device staging buffers per tensor shape, {args.e2e_chunks} batch slice(s) per call",
                "link_gbs_both_directions_busy": r["link"]},
        "e2e_fp32_activations": {"value": e2e32, "unit": "img/s", "h2d_bytes_per_step": r["h2d32"],
                                 "d2h_bytes_per_step": r["d2h"]},
        "gpu_launches": r["launches"],
        "clocks": r["clocks"],
        "roofline": dominant,
        "roofline_secondary": secondary if secondary["launches_per_step"] else roof_expand,
        "roofline_pointwise": r["pw"],
        "roofline_caller_passes": [
            {"bound": "hbm", "kernel": "counts_to_value_kernel<half> (int16 counts -> fp16 values, both signs)",
             "achieved": r["c2v_gbs"], "unit": "GB/s", "peak": _hbm_peak(), "frac": r["c2v_gbs"] / _hbm_peak(),
             "peak_source": _hbm_peak_source()},
            {"bound": "hbm", "kernel": "max_count_kernel + calib_bins_kernel<float> (calibration window statistics)",
             "achieved": r["calib_gbs"], "unit": "GB/s", "peak": _hbm_peak(), "frac": r["calib_gbs"] / _hbm_peak(),
             "peak_source": _hbm_peak_source()},
        ],
        "per_layer": r["per_layer"],
    }
    if secondary["launches_per_step"]:
        line["roofline_expand"] = roof_expand
    return line


# ---- SC linear -------------------------------------------------------------------------------------------------
def run_linear(args, wl, rank, world, local_rank):
    from rexsc_b200 import _lib, ops, sharding

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    g = torch.Generator().manual_seed(3 + rank)
    B = wl["batch"]
    data = []
    for cin, cout, L in wl["layers"]:
        x = ((torch.rand(B, cin, generator=g) * 128).round().clamp(0, 127) / 128).to(dev)
        w = (((torch.randn(cout, cin, generator=g) * 0.1).clamp(-1, 1) * 128).round() / 128).to(dev)
        data.append((x, w, L))

    def step():
        for x, w, L in data:
            ops.linear_generic_general_acc(x, w, PROG, L, -1, wl["or_n"] - 1, 1, True, False)

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    c0 = _lib.load().rexsc_kernel_launch_count()
    ms = _timed_steps(step, args.steps, args.warmup, world, dev, sharding)
    n_launch = (_lib.load().rexsc_kernel_launch_count() - c0) * args.steps // (args.steps + args.warmup)
    clocks = sampler.stop() if rank == 0 else None
    pins = [(x.cpu().pin_memory(), w, L) for x, w, L in data]

    outs_pin = [(torch.empty(B, w.shape[0], dtype=torch.int16).pin_memory(),
                 torch.empty(B, w.shape[0], dtype=torch.int16).pin_memory()) for _, w, _ in data]

    def step_host():
        for (xh, w, L), (ph, nh) in zip(pins, outs_pin):
            p, n = ops.linear_generic_general_acc(xh.to(dev, non_blocking=True), w, PROG, L, -1, wl["or_n"] - 1, 1,
                                                  True, False)
            ph.copy_(p, non_blocking=True)
            nh.copy_(n, non_blocking=True)
        return outs_pin

    e2e_steps = max(1, min(args.steps, 5))
    ms_e2e = _timed_steps(step_host, e2e_steps, 1, world, dev, sharding)
    bitops = sum(2 * L * B * cin * cout for cin, cout, L in wl["layers"])
    return {"ms": ms, "ms_e2e": ms_e2e, "e2e_steps": e2e_steps, "clocks": clocks, "bitops": bitops, "launches": n_launch,
            "h2d": sum(x.numel() * 4 for x, _, _ in data), "d2h": sum(2 * 2 * B * cout for _, cout, _ in wl["layers"])}


def linear_line(args, wl, r, world):
    B = wl["batch"]
    value = B * world * args.steps / (r["ms"] * 1e-3)
    return {
        "metric": wl["metric"], "value": value, "unit": "rows/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": r["ms"] / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "u32 bit-streams / int16 sums", "data": "synthetic",
        "config": {"workload": wl["text"], "batch_per_gpu": B,
                   "l2_policy": "working set (< 1 MB) is cache resident by nature: the op is launch-latency bound"},
        "tbitops_per_s": r["bitops"] * world * args.steps / (r["ms"] * 1e-3) / 1e12,
        "e2e": {"value": B * world * r["e2e_steps"] / (r["ms_e2e"] * 1e-3), "unit": "rows/s",
                "h2d_bytes_per_step": r["h2d"], "d2h_bytes_per_step": r["d2h"]},
        "gpu_launches": r["launches"], "clocks": r["clocks"],
        "roofline": {"bound": "latency", "kernel": "SC linear = SC conv with 1x1 geometry",
                     "achieved": r["ms"] / args.steps / len(wl["layers"]) * 1e3, "unit": "us per layer call",
                     "peak": None, "frac": None, "traffic": None},
    }


# ---- FXP conv ---------------------------------------------------------------------------------------------------
def run_fxp(args, wl, rank, world, local_rank):
    from rexsc_b200 import _lib, ops, sharding

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    g = torch.Generator().manual_seed(1 + rank)
    B = wl["batch"]
    data = []
    for cin, h, cout, k, p, pin in wl["layers"]:
        x = torch.rand(B, cin, h, h, generator=g).to(dev)
        w = (torch.randn(cout, cin, k, k, generator=g) * 0.1).clamp(-1, 1).to(dev)
        data.append((x, w, p, pin))

    def step():
        for x, w, p, pin in data:
            ops.conv2d_saturate_acc(x, w, 0, pin, 24, (p, p), (1, 1))

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    c0 = _lib.load().rexsc_kernel_launch_count()
    ms = _timed_steps(step, args.steps, args.warmup, world, dev, sharding)
    n_launch = (_lib.load().rexsc_kernel_launch_count() - c0) * args.steps // (args.steps + args.warmup)
    clocks = sampler.stop() if rank == 0 else None
    pins = [(x.cpu().pin_memory(), w, p, pin) for x, w, p, pin in data]

    # pinned host buffers for the results too: a pageable `.cpu()` copy would synchronise and crawl
    outs_pin = [torch.empty_like(ops.conv2d_saturate_acc(x, w, 0, pin, 24, (p, p), (1, 1)), device="cpu").pin_memory()
                for x, w, p, pin in data]

    def step_host():
        for (xh, w, p, pin), oh in zip(pins, outs_pin):
            oh.copy_(ops.conv2d_saturate_acc(xh.to(dev, non_blocking=True), w, 0, pin, 24, (p, p), (1, 1)),
                     non_blocking=True)
        return outs_pin

    e2e_steps = max(1, min(args.steps, 5))
    ms_e2e = _timed_steps(step_host, e2e_steps, 1, world, dev, sharding)
    per_layer, total_ops = [], 0.0
    for (x, w, p, pin), (cin, h, cout, k, _, _) in zip(data, wl["layers"]):
        t = _event_ms(lambda: ops.conv2d_saturate_acc(x, w, 0, pin, 24, (p, p), (1, 1)))
        oh = h + 2 * p - k + 1
        # int8 ops of the closed form: values and parity bits, positive and negative weights, multiply + add
        intops = 2.0 * 2 * 2 * B * oh * oh * cout * cin * k * k
        total_ops += intops
        per_layer.append({"shape": [cin, h, cout, k, p, pin], "ms": round(t, 4), "int8_tops": round(intops / t / 1e9, 1)})
    return {"ms": ms, "ms_e2e": ms_e2e, "e2e_steps": e2e_steps, "clocks": clocks, "per_layer": per_layer,
            "launches": n_launch, "intops": total_ops, "mma_peak_ops": _mma_peak(ops, dev), "h2d": sum(x.numel() * 4 for x, _, _, _ in data),
            "d2h": sum(4 * B * cout * (h + 2 * p - k + 1) ** 2 for cin, h, cout, k, p, pin in wl["layers"])}


def fxp_line(args, wl, r, world):
    B = wl["batch"]
    value = B * world * args.steps / (r["ms"] * 1e-3)
    kernel_ms = sum(l["ms"] for l in r["per_layer"])
    achieved = r["intops"] / (kernel_ms * 1e-3)
    return {
        "metric": wl["metric"], "value": value, "unit": "img/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": r["ms"] / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8 operands / int32 accumulators (24-bit saturation)", "data": "synthetic",
        "config": {"workload": wl["text"], "batch_per_gpu": B,
                   "l2_policy": "working set (< 40 MB) fits L2: small-layer workload, reported as such"},
        "e2e": {"value": B * world * r["e2e_steps"] / (r["ms_e2e"] * 1e-3), "unit": "img/s",
                "h2d_bytes_per_step": r["h2d"], "d2h_bytes_per_step": r["d2h"]},
        "gpu_launches": r["launches"], "clocks": r["clocks"],
        "roofline": {"bound": "tensor", "kernel": "fxp_conv_umma_kernel (tcgen05 int8 closed form) + operand packing",
                     "achieved": achieved / 1e12, "peak": r["mma_peak_ops"] / 1e12, "unit": "TOP/s int8",
                     "frac": achieved / r["mma_peak_ops"], "traffic": None, "kernel_ms_per_step": kernel_ms,
                     "peak_source": "measured live: back-to-back tcgen05.mma kind::i8 probe on this GPU"},
        "per_layer": r["per_layer"],
    }


# ---- training step through the reference's own loop ---------------------------------------------------------------
def run_train(args, rank, world, local_rank):
    """Training-step throughput (the first half of the headline metric): the reference's own models and training loop
    on the drop-in ops, synthetic ImageNet-shaped batches, per `sync` mode; with several GPUs the weight gradients
    are all-reduced over NCCL inside the timed region.  Every rank takes part; the numbers are whole-job."""
    from rexsc_b200 import ops

    ops.release_workspaces()
    torch.cuda.empty_cache()
    try:
        from rexsc_b200 import frontend
        from rexsc_b200.frontend import train as fe_train

        fe = frontend.load()
    except ImportError as exc:
        return {"unavailable": str(exc).splitlines()[0]}
    ops.manual_seed(0, rank)
    return fe_train.train_block(args.train_workload, warmup=max(10, args.train_warmup), steps=args.train_steps,
                                device=torch.device("cuda", local_rank), rank=rank, world=world, fe=fe)


# ---- the reference's CPU implementation (cpu_baseline and --impl reference) -----------------------------------------
_REF_CPU = {}


def load_reference_cpu():
    """The reference's own CPU extensions from oracle/_ref (built by oracle/build_ref.py); None if they cannot run
    on this host.  Probed once per process, outside every timed region."""
    if "mods" not in _REF_CPU:
        _REF_CPU["mods"] = _load_reference_cpu()
    return _REF_CPU["mods"]


def _load_reference_cpu():
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import build_ref

    so = os.path.join(ROOT, "oracle", "_ref", "sc_extension_ref.so")
    if not os.path.exists(so):
        return None
    # the extension was compiled with -march=native elsewhere: prove in a child process that it runs here
    probe = ("import sys, torch; sys.path.insert(0, %r); import build_ref; m = build_ref.load(); "
             "x = torch.rand(1, 8, 6, 6); w = torch.rand(8, 8, 3, 3) - 0.5; "
             "m[0].conv2d_generic_general(x, w, 32, -1, 16, (1, 1), (1, 1), (7, 8, 1), 1, 1, False, False)"
             % os.path.join(ROOT, "oracle"))
    try:
        if subprocess.run([sys.executable, "-c", probe], capture_output=True, timeout=300).returncode != 0:
            return None
        return build_ref.load()
    except Exception:
        return None


def cpu_reference_time(wl, batch, threads):
    """(seconds, kind) for one pass of the workload's layers at `batch` through the reference CPU extension
    (XOR-LFSR semantics: the only ones that code has), or through the oracle port when the extension cannot run."""
    mods = load_reference_cpu()
    kind = "reference"
    if mods is None:
        sys.path.insert(0, os.path.join(ROOT, "oracle"))
        import oracle as port

        kind = "port"
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(5)
    total = 0.0
    if wl["kind"] == "sc":
        fmt = torch.channels_last if wl["channels_last"] else torch.contiguous_format
        for cin, h, cout, k, s, p, rep, L in wl["layers"]:
            x = torch.rand(batch, cin, h, h, generator=g).contiguous(memory_format=fmt)
            w = (torch.randn(cout, cin, k, k, generator=g) * 0.1).clamp(-1, 1).contiguous(memory_format=fmt)
            a = (x, w, L, -1, 16, (p, p), (s, s), PROG, wl["or_n"] - 1, 1, False, False)
            t0 = time.perf_counter()
            mods[0].conv2d_generic_general(*a) if kind == "reference" else port.conv2d_generic_general_split(*a)
            total += (time.perf_counter() - t0) * rep
    elif wl["kind"] == "fxp":
        for cin, h, cout, k, p, pin in wl["layers"]:
            x = torch.rand(batch, cin, h, h, generator=g)
            w = (torch.randn(cout, cin, k, k, generator=g) * 0.1).clamp(-1, 1)
            a = (x, w, 0, pin, 24, (p, p), (1, 1))
            t0 = time.perf_counter()
            mods[1].conv2d_saturate(*a) if kind == "reference" else port.conv2d_saturate(*a)
            total += time.perf_counter() - t0
    else:  # linear; the reference's CPU linear reads rows in blocks of 128 (sc_matmul.cpp:428-438): keep multiples
        for cin, cout, L in wl["layers"]:
            co = (cout + 127) // 128 * 128
            x = torch.rand(batch, cin, generator=g)
            w = (torch.randn(co, cin, generator=g) * 0.1).clamp(-1, 1)
            a = (x, w, PROG, L, -1, wl["or_n"] - 1, 1, False, False)
            t0 = time.perf_counter()
            mods[0].linear_generic_general(*a) if kind == "reference" else port.linear_generic_general(*a)
            total += time.perf_counter() - t0
    return total, kind


def _sample_batch(wl):
    """Batch of a bounded CPU sample: about what batch 4 of the ResNet-18 workload costs (a few seconds per pass)."""
    if wl["kind"] == "sc":
        work = bitops_per_image(wl["layers"])
        return max(1, min(wl["batch"], int(4.2 * 1.085e11 / work)))
    return wl["batch"] if wl["kind"] == "fxp" else 128


def cpu_baseline_block(wl):
    threads = os.cpu_count() or 1
    os.environ.setdefault("OMP_NUM_THREADS", str(threads))
    sb = _sample_batch(wl)
    load_reference_cpu()
    secs, kind = cpu_reference_time(wl, sb, threads)
    unit = "rows/s" if wl["kind"] == "linear" else "img/s"
    return {"value": sb / secs, "unit": unit, "cores": threads, "kind": kind,
            "sample": f"every layer of the workload at batch {sb} (of {wl['batch']}), one pass, {secs:.1f} s; "
                      "the CPU code has no XNOR generator (xnor=False) and no point-wise ops"}


def run_reference(args, wl, rank, world):
    if rank != 0:
        return None
    threads = os.cpu_count() or 1
    os.environ.setdefault("OMP_NUM_THREADS", str(threads))
    sb = _sample_batch(wl)
    load_reference_cpu()
    if args.warmup > 0:
        cpu_reference_time(dict(wl, layers=wl["layers"][-1:]), sb, threads)
    t0 = time.perf_counter()
    kind = "reference"
    for _ in range(args.steps):
        _, kind = cpu_reference_time(wl, sb, threads)
    dt = time.perf_counter() - t0
    value = sb * args.steps / dt
    unit = "rows/s" if wl["kind"] == "linear" else "img/s"
    sample = f"every layer of the workload at batch {sb} per step on the host cores, xnor=False"
    return {
        "impl": "reference", "metric": wl["metric"], "value": value, "unit": unit,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u32 bit-streams / int16",
        "data": "synthetic",
        # the same workload description as the other arm; what a step samples of it is in cpu_baseline.sample
        "config": {"workload": wl["text"], "batch_per_gpu": wl["batch"]},
        "cpu_baseline": {"value": value, "unit": unit, "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="resnet18", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-train", action="store_true", help="skip the training-step block")
    ap.add_argument("--train-steps", type=int, default=30)
    ap.add_argument("--train-warmup", type=int, default=10)
    ap.add_argument("--train-workload", default=None)
    ap.add_argument("--e2e-slots", type=int, default=6,
                    help="host-buffer leg: device staging buffers per tensor shape (how far copies may run ahead)")
    ap.add_argument("--e2e-chunks", type=int, default=1,
                    help="host-buffer leg: run every conv call as this many calls on slices of its batch")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    wl = WORKLOADS[args.config]
    args.train_workload = args.train_workload or TRAIN_WORKLOAD.get(args.config)

    if args.impl == "reference":
        args.steps = args.steps if args.steps is not None else 2
        args.warmup = args.warmup if args.warmup is not None else 1
        line = run_reference(args, wl, rank, world)
        if line is not None:
            print(json.dumps(line), flush=True)
        return

    args.steps = args.steps if args.steps is not None else 10
    args.warmup = max(3, args.warmup if args.warmup is not None else 3)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the rexsc_b200 hot path has no CPU fallback")
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    runner, liner = {"sc": (run_sc, sc_line), "linear": (run_linear, linear_line), "fxp": (run_fxp, fxp_line)}[wl["kind"]]
    r = runner(args, wl, rank, world, local_rank)
    if world > 1:
        torch.distributed.barrier()
    train = None
    if not args.no_train and args.train_workload is not None:
        train = run_train(args, rank, world, local_rank)
    if rank == 0:
        line = liner(args, wl, r, world)
        if train is not None:
            line["train"] = train
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_block(wl)
        print(json.dumps(line), flush=True)
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
