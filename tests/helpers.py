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


def reference_gpu_modules():
    """(sc_extension_cuda_ref, fixed_extension_cuda_ref) built by oracle/build_ref.py --gpu, or None."""
    import build_ref

    try:
        return build_ref.load_gpu()
    except Exception:  # built for another torch / CUDA runtime
        return None


class ops_of:
    """Context manager: inside it the reference's utils_functional calls ``mods`` (e.g. the reference's own GPU
    extensions) instead of the drop-in modules it imported.  Only the two module-level names of
    utils_functional.py:18,20 are rebound; nothing of the front end's code changes."""

    def __init__(self, fe, mods):
        self.uf, self.mods = fe.utils_functional, mods

    def __enter__(self):
        self.saved = (self.uf.sc_extension_cuda, self.uf.fixed_extension_cuda)
        self.uf.sc_extension_cuda, self.uf.fixed_extension_cuda = self.mods
        return self

    def __exit__(self, *exc):
        self.uf.sc_extension_cuda, self.uf.fixed_extension_cuda = self.saved
        return False


def rel_err(a, b):
    """max |a - b| / max |b| over two tensors (the relative measure used for gradients)."""
    a, b = a.detach().double(), b.detach().double()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))
