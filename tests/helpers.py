"""Shared helpers of the test-suite: seeded inputs in the reference's value distributions and fixture access."""
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def quantize(t, prec):
    # forward part of the reference's quantiser (utils_functional.py:93-123)
    s = 2 ** prec
    return (t * s).round().clamp(-s + 1, s - 1) / s


def conv_inputs(N, Cin, H, W, Cout, K, prec=7, seed=0, wscale=0.1, KW=None):
    g = torch.Generator().manual_seed(seed)
    x = quantize(torch.rand(N, Cin, H, W, generator=g), prec)
    w = quantize((torch.randn(Cout, Cin, K, KW or K, generator=g) * wscale).clamp(-1, 1), prec)
    return x, w


def load_golden(name):
    return np.load(os.path.join(GOLDEN, name))


def golden_cases(npz):
    return sorted({k.split("/")[0] for k in npz.files})


def from128(a):
    return torch.from_numpy(a.astype(np.float32) / 128.0)


def checksum(a: np.ndarray) -> int:
    a = a.astype(np.int64).reshape(-1)
    idx = (np.arange(a.size, dtype=np.int64) % 65521) + 1
    return int((a * idx).sum())
