"""Time the reference's own GPU extensions (compiled unchanged for sm_100 by ``oracle/build_ref.py --gpu``) next
to this library on the same inputs: the "kernel to beat".  Test infrastructure, not part of the product.

    python oracle/time_ref_gpu.py            # on a GPU box; prints one line per case

The reference's linear op is never called (it faults after a conv in the same process, see
tests/test_gpu_vs_reference_gpu_ext.py)."""
from __future__ import annotations

import json
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))
import build_ref  # noqa: E402

PROG = (7, 8, 1)


def timed(fn, reps=3):
    fn()
    torch.cuda.synchronize()
    best = None
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        t = e0.elapsed_time(e1)
        best = t if best is None else min(best, t)
    return best


def main():
    from rexsc_b200 import ops

    mods = build_ref.load_gpu()
    if mods is None:
        raise SystemExit("oracle/_ref holds no reference GPU extension")
    sc, fx = mods
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(0)
    rows = []
    # (N, Cin, H (unpadded), Cout, K, stride, pad, L, or_n, channels_last)
    convs = [(256, 64, 56, 64, 3, 1, 1, 32, 2, True), (256, 64, 56, 128, 3, 2, 1, 32, 2, True),
             (256, 128, 28, 128, 3, 1, 1, 32, 2, True), (256, 256, 14, 256, 3, 1, 1, 32, 2, True),
             (256, 512, 7, 512, 3, 1, 1, 32, 2, True), (256, 64, 56, 128, 1, 2, 0, 32, 2, True),
             (192, 64, 56, 64, 3, 1, 1, 64, 3, True), (32, 3, 32, 32, 5, 1, 2, 32, 1, False),
             (256, 64, 32, 64, 3, 1, 1, 32, 1, False)]
    for N, C, H, Co, K, s, p, L, or_n, cl in convs:
        x = torch.rand(N, C, H + 2 * p, H + 2 * p, device=dev, generator=g)
        w = (torch.randn(Co, C, K, K, device=dev, generator=g) * 0.1).clamp(-1, 1)
        if cl:
            x = x.contiguous(memory_format=torch.channels_last)
            w = w.contiguous(memory_format=torch.channels_last)
        args = (L, -1, 16, (0, 0), (s, s), PROG, or_n - 1, 1, True, False)
        t_ref = timed(lambda: sc.conv2d_generic_general_split_acc(x, w, *args))
        t_our = timed(lambda: ops.conv2d_generic_general_split_acc(x, w, *args))
        rp, rn = sc.conv2d_generic_general_split_acc(x, w, *args)
        p_, n_ = ops.conv2d_generic_general_split_acc(x, w, *args)
        same = bool(torch.equal(rp, p_) and torch.equal(rn, n_))
        oh = (H + 2 * p - K) // s + 1
        bitops = 2 * L * N * oh * oh * Co * C * K * K
        rows.append({"op": "sc_conv", "shape": [N, C, H, Co, K, s, L, or_n], "ref_ms": t_ref, "ours_ms": t_our,
                     "speedup": t_ref / t_our, "ref_tbitops": bitops / t_ref / 1e9, "ours_tbitops": bitops / t_our / 1e9,
                     "bit_exact": same})
        print(json.dumps(rows[-1]), flush=True)
    # point-wise ops on a ResNet-18 layer-1 sized tensor
    s_ = (torch.rand(256, 64, 56, 56, device=dev, generator=g) * 4).contiguous(memory_format=torch.channels_last)
    s16 = s_.half()
    grad = torch.randn_like(s_)
    bias = torch.tensor([0.01, -0.05, 0.02, 0.003, -0.001, 0.0002, 0, 0, 0, 0, 0], device=dev)
    std = torch.tensor([0.02, 0.05, -0.01, 0.002, 0.0, 0.0001, 0, 0, 0, 0, 0], device=dev)
    n_el = s_.numel()
    pw = [("orn_fwd_f16in", lambda m: m.or_approx_n_forward_acc(s16, 2), 6),
          ("orn_bwd_f16in", lambda m: m.or_approx_n_backward_acc(grad, s16, 2), 10),
          ("both_fwd_f16in", lambda m: m.or_approx_n_forward_bias_std_both_acc(s16, s16, bias, std, 2), 8),
          ("both_bwd_f16in", lambda m: m.or_approx_n_backward_bias_std_both_acc(grad, s16, s16, bias, 2), 16)]
    for name, fn, bytes_per in pw:
        t_ref = timed(lambda: fn(sc))
        t_our = timed(lambda: fn(ops))
        rows.append({"op": name, "elements": n_el, "ref_ms": t_ref, "ours_ms": t_our, "speedup": t_ref / t_our,
                     "ref_gbs": n_el * bytes_per / t_ref / 1e6, "ours_gbs": n_el * bytes_per / t_our / 1e6})
        print(json.dumps(rows[-1]), flush=True)
    # FXP conv, TinyConv layers at batch 256
    for N, C, H, Co, K, p, pin in [(256, 3, 32, 32, 5, 2, 5), (256, 32, 16, 32, 5, 2, 5), (256, 32, 8, 64, 5, 2, 5),
                                   (256, 64, 4, 10, 4, 0, 7)]:
        x = torch.rand(N, C, H, H, device=dev, generator=g)
        w = (torch.randn(Co, C, K, K, device=dev, generator=g) * 0.1).clamp(-1, 1)
        t_ref = timed(lambda: fx.conv2d_saturate_acc(x, w, 0, pin, 24, (p, p), (1, 1)))
        t_our = timed(lambda: ops.conv2d_saturate_acc(x, w, 0, pin, 24, (p, p), (1, 1)))
        same = bool(torch.equal(fx.conv2d_saturate_acc(x, w, 0, pin, 24, (p, p), (1, 1)),
                                ops.conv2d_saturate_acc(x, w, 0, pin, 24, (p, p), (1, 1))))
        rows.append({"op": "fxp_conv", "shape": [N, C, H, Co, K], "ref_ms": t_ref, "ours_ms": t_our,
                     "speedup": t_ref / t_our, "bit_exact": same})
        print(json.dumps(rows[-1]), flush=True)


if __name__ == "__main__":
    main()
