"""Generate tests/golden/*.npz by EXECUTING the reference's own CPU extensions.

Run in a container that has the reference checkout:
    python oracle/build_ref.py && python tests/golden/make_golden.py

Each fixture stores the seeded inputs (so a different torch RNG cannot shift
them; every input is a multiple of 1/128 and is stored as int16 = value*128), the
op arguments and the reference output.  The reference CPU extension
implements the XOR-feedback LFSR only and returns pos-neg for conv
(torch_c/sc-extension/sc_conv.cpp:301-489), int32 pos/neg for linear
(sc_matmul.cpp:576-676) and int32 for the FXP conv (fixed.cpp:197-238).
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
import build_ref  # noqa: E402


def quantize(t, prec):
    # utils_functional.py:93-123 (forward part): clamp(round(x*2^p), -2^p+1, 2^p-1) / 2^p
    s = 2 ** prec
    return (t * s).round().clamp(-s + 1, s - 1) / s


def checksum(a: np.ndarray) -> int:
    a = a.astype(np.int64).reshape(-1)
    idx = (np.arange(a.size, dtype=np.int64) % 65521) + 1
    return int((a * idx).sum())


CONV_CASES = [
    # name, N, Cin, H, W, Cout, K, pad, stride, L, or_n, channels_last, prec, seed
    ("cfg1_or1_L32", 32, 3, 32, 32, 32, 5, 2, 1, 32, 1, False, 5, 0),
    ("cfg1_or2_L32", 32, 3, 32, 32, 32, 5, 2, 1, 32, 2, False, 5, 0),
    ("cfg1_or3_L64", 32, 3, 32, 32, 32, 5, 2, 1, 64, 3, False, 5, 0),
    ("c32_k3_or2_L32_cl", 2, 32, 10, 10, 16, 3, 1, 1, 32, 2, True, 7, 3),
    ("c70_k3_s2_or2_L32", 2, 70, 9, 9, 40, 3, 1, 2, 32, 2, False, 5, 2),
    ("c64_k1_s2_or3_L64_cl", 3, 64, 8, 8, 24, 1, 0, 2, 64, 3, True, 7, 4),
    ("c16_k4_or1_L128", 2, 16, 4, 4, 10, 4, 0, 1, 128, 1, False, 7, 5),
    ("c5_k5_or4_L32", 1, 5, 12, 7, 7, 5, 2, 1, 32, 4, False, 5, 6),
    ("c40_k3_fullbin_L32", 1, 40, 6, 6, 9, 3, 1, 1, 32, 51201, False, 5, 7),
    ("c8_k3_or1_L16", 2, 8, 6, 6, 5, 3, 1, 1, 16, 1, False, 4, 8),
    ("c8_k3_or2_L8", 2, 8, 6, 6, 5, 3, 1, 1, 8, 2, False, 3, 9),
]


def make_conv(sc):
    out = {}
    for name, N, Cin, H, W, Cout, K, pad, stride, L, or_n, cl, prec, seed in CONV_CASES:
        torch.manual_seed(seed)
        x = quantize(torch.rand(N, Cin, H, W), prec)
        w = quantize((torch.randn(Cout, Cin, K, K) * 0.1).clamp(-1, 1), prec)
        xi, wi = x, w
        if cl:
            xi = x.contiguous(memory_format=torch.channels_last)
            wi = w.contiguous(memory_format=torch.channels_last)
        y = sc.conv2d_generic_general(xi, wi, L, -1, 16, (pad, pad), (stride, stride), (7, 8, 1), or_n - 1, 1,
                                      False, False)
        y = y.contiguous().numpy()
        full = y.size <= 70000
        out[name + "/x128"] = (x * 128).round().to(torch.int16).numpy()
        out[name + "/w128"] = (w * 128).round().to(torch.int16).numpy()
        out[name + "/args"] = np.array([N, Cin, H, W, Cout, K, pad, stride, L, or_n, int(cl)], dtype=np.int64)
        out[name + "/sum"] = np.array([int(y.astype(np.int64).sum()), checksum(y)], dtype=np.int64)
        if full:
            out[name + "/y"] = y
        else:
            out[name + "/y_head"] = y.reshape(-1)[:4096].copy()
        print(name, "sum", out[name + "/sum"], "full" if full else "head")
    np.savez_compressed(os.path.join(HERE, "sc_conv_ref_cpu.npz"), **out)


LINEAR_CASES = [
    # name, B, Cin, Cout, L, or_n, seed   (B and Cout multiples of 128: the CPU kernel reads whole blocks)
    ("b128_c512_o128_L32_or1", 128, 512, 128, 32, 1, 10),
    ("b128_c1024_o128_L128_or2", 128, 1024, 128, 128, 2, 11),
    ("b256_c70_o256_L32_or3", 256, 70, 256, 32, 3, 12),
]


def make_linear(sc):
    out = {}
    for name, B, Cin, Cout, L, or_n, seed in LINEAR_CASES:
        torch.manual_seed(seed)
        x = quantize(torch.rand(B, Cin), 7)
        w = quantize((torch.randn(Cout, Cin) * 0.1).clamp(-1, 1), 7)
        p, n = sc.linear_generic_general(x, w, (7, 8, 1), L, -1, or_n - 1, 1, False, False)
        out[name + "/x128"] = (x * 128).round().to(torch.int16).numpy()
        out[name + "/w128"] = (w * 128).round().to(torch.int16).numpy()
        out[name + "/args"] = np.array([B, Cin, Cout, L, or_n], dtype=np.int64)
        out[name + "/pos"] = p.numpy().astype(np.int16)
        out[name + "/neg"] = n.numpy().astype(np.int16)
        print(name, int(p.sum()), int(n.sum()))
    np.savez_compressed(os.path.join(HERE, "sc_linear_ref_cpu.npz"), **out)


FXP_CASES = [
    # name, N, Cin, H, W, Cout, K, pad, stride, add_config, p_in, p_out, wscale, seed
    ("tiny1_3to32_k5", 2, 3, 32, 32, 32, 5, 2, 1, 0, 5, 24, 0.1, 1),
    ("tiny2_32to32_k5", 2, 32, 16, 16, 32, 5, 2, 1, 0, 5, 24, 0.1, 1),
    ("tiny3_32to64_k5", 2, 32, 8, 8, 64, 5, 2, 1, 0, 5, 24, 0.1, 1),
    ("tiny4_64to10_k4_p7", 4, 64, 4, 4, 10, 4, 0, 1, 0, 7, 24, 0.1, 1),
    ("sat_cap_p7_out16", 1, 16, 6, 6, 8, 3, 1, 1, 0, 7, 16, 0.15, 20),  # K = 144 (multiple of 8), cap 2^16 reached by some
    ("shift_p7_out10", 1, 16, 6, 6, 8, 3, 1, 1, 0, 7, 10, 0.02, 21),    # precision_diff = 4, K = 144
    ("oradd_p5", 1, 16, 6, 6, 8, 3, 1, 1, 1, 5, 24, 0.1, 22),
    ("or2add_p5", 1, 16, 6, 6, 8, 3, 1, 1, 2, 5, 24, 0.1, 23),
    ("stride2_p5", 2, 8, 9, 9, 6, 3, 1, 2, 0, 5, 24, 0.3, 24),
]


def make_fxp(fx):
    out = {}
    for name, N, Cin, H, W, Cout, K, pad, stride, add, p_in, p_out, ws, seed in FXP_CASES:
        torch.manual_seed(seed)
        x = quantize(torch.rand(N, Cin, H, W), 7)
        w = quantize((torch.randn(Cout, Cin, K, K) * ws).clamp(-1, 1), 7)
        y = fx.conv2d_saturate(x, w, add, p_in, p_out, (pad, pad), (stride, stride)).numpy()
        out[name + "/x128"] = (x * 128).round().to(torch.int16).numpy()
        out[name + "/w128"] = (w * 128).round().to(torch.int16).numpy()
        out[name + "/args"] = np.array([N, Cin, H, W, Cout, K, pad, stride, add, p_in, p_out], dtype=np.int64)
        out[name + "/y"] = y
        print(name, int(y.astype(np.int64).sum()), int(y.max()), int(y.min()))
    np.savez_compressed(os.path.join(HERE, "fxp_conv_ref_cpu.npz"), **out)


if __name__ == "__main__":
    if not build_ref.build():
        raise SystemExit("reference sources not available: cannot regenerate the golden vectors")
    sc, fx = build_ref.load()
    torch.set_num_threads(1)
    make_conv(sc)
    make_linear(sc)
    make_fxp(fx)
