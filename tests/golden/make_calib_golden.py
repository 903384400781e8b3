"""Generate tests/golden/calib_ref_py.npz by EXECUTING the reference's own compute_bias_std_coef
(utils_functional.py:901-950) on CPU tensors.

Run in a container that has the reference checkout (its path in REXSC_REFERENCE_ROOT, as for oracle/build_ref.py):
    python tests/golden/make_calib_golden.py

The reference module imports its four extension modules at load time; the stand-in modules of
rexsc_b200.install_dropin() satisfy those imports (none of them is called by compute_bias_std_coef).  The
per-window bias / std values the function fits are captured from its two torch.linalg.lstsq calls.  Each case
stores the int16 counts, the fp32 guide values, L, and the reference's windows, per-window statistics and
coefficients.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

# name, elements per sign, L, or_n, guide range, noise, seed
CASES = [
    ("or2_L32", 6000, 32, 2, 1.9, 0.03, 0),
    ("or3_L64", 5000, 64, 3, 2.7, 0.04, 1),
    ("or1_L32_sparse", 300, 32, 1, 0.9, 0.08, 2),   # several windows hold fewer than two elements
    ("or2_L128_narrow", 4000, 128, 2, 0.25, 0.02, 3),  # windows overlap heavily (spacing far below 0.1)
]


def inputs(n, L, or_n, hi, noise, seed):
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(2):
        act = torch.rand(n, generator=g) ** 2 * hi
        cnt = torch.round((act * (1 - 0.04 * act) + noise * torch.randn(n, generator=g)) * L).clamp(0, or_n * L)
        out += [cnt.to(torch.int16), act.float()]
    return out  # pos, value_pos, neg, value_neg


def main():
    from rexsc_b200 import frontend

    # the reference's utils_functional from its checkout (REXSC_REFERENCE_ROOT or BASELINE.json's reference_path)
    if frontend.reference_root() is None:
        raise SystemExit("make_calib_golden: no reference checkout reachable (set REXSC_REFERENCE_ROOT)")
    uf = frontend.load().utils_functional

    real_lstsq = torch.linalg.lstsq
    out = {}
    for name, n, L, or_n, hi, noise, seed in CASES:
        pos, vpos, neg, vneg = inputs(n, L, or_n, hi, noise, seed)
        a_bit = torch.cat([pos.float() / L, neg.float() / L])
        a_act = torch.cat([vpos, vneg])
        seen = []

        def spy(a, b, *args, **kw):
            seen.append((a.clone(), b.clone()))
            return real_lstsq(a, b, *args, **kw)

        torch.linalg.lstsq = spy
        try:
            bias_coef, std_coef = uf.compute_bias_std_coef(or_n, a_bit, a_act, 5)
        finally:
            torch.linalg.lstsq = real_lstsq
        basis, std_bins = seen[-1]
        out[f"{name}/pos"] = pos.numpy()
        out[f"{name}/neg"] = neg.numpy()
        out[f"{name}/value_pos"] = vpos.numpy()
        out[f"{name}/value_neg"] = vneg.numpy()
        out[f"{name}/args"] = np.array([L, or_n], dtype=np.int64)
        out[f"{name}/starts"] = basis[:, 1].numpy()      # the valid window starts (column x^1 of the basis)
        out[f"{name}/std_bins"] = std_bins.numpy()
        if len(seen) == 2:
            out[f"{name}/bias_bins"] = seen[0][1].numpy()
        out[f"{name}/bias_coef"] = bias_coef.numpy()
        out[f"{name}/std_coef"] = std_coef.numpy()
        print(name, "valid windows", basis.shape[0], "bias fitted", len(seen) == 2)
    path = os.path.join(HERE, "calib_ref_py.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
