"""CPU tests: the oracle's restatement of the calibration statistics (compute_bias_std_coef,
utils_functional.py:901-950) against vectors produced by the reference's own function
(tests/golden/calib_ref_py.npz, made by tests/golden/make_calib_golden.py).

Tolerance: the reference reduces in fp32 (torch mean / std), the oracle in float64; per-window values agree to
1e-5 relative + 1e-6 absolute.  Fitted polynomials are compared by value over the fitted range (1e-3 absolute),
not coefficient by coefficient: the degree-5 normal equations are ill-conditioned."""
import numpy as np
import torch

from helpers import golden_cases, load_golden


def _case(npz, name):
    g = {k.split("/", 1)[1]: npz[k] for k in npz.files if k.startswith(name + "/")}
    L, or_n = (int(v) for v in g["args"])
    return g, L, or_n


def test_calib_windows_match_reference_function(oracle):
    npz = load_golden("calib_ref_py.npz")
    for name in golden_cases(npz):
        g, L, or_n = _case(npz, name)
        a_bit = np.concatenate([g["pos"], g["neg"]]).astype(np.float32) / L
        a_act = np.concatenate([g["value_pos"], g["value_neg"]])
        starts, count, mean, std = oracle.calib_windows(a_bit, a_act)
        valid = count > 1
        assert np.allclose(starts[valid].astype(np.float32), g["starts"], rtol=1e-6, atol=0), name
        assert np.allclose(std[valid], g["std_bins"], rtol=1e-5, atol=1e-6), name
        if "bias_bins" in g:
            assert np.allclose(mean[valid], g["bias_bins"], rtol=1e-5, atol=1e-6), name


def test_calib_fit_matches_reference_function(oracle):
    npz = load_golden("calib_ref_py.npz")
    for name in golden_cases(npz):
        g, L, or_n = _case(npz, name)
        a_bit = torch.from_numpy(np.concatenate([g["pos"], g["neg"]]).astype(np.float32) / L)
        a_act = torch.from_numpy(np.concatenate([g["value_pos"], g["value_neg"]]))
        bias_coef, std_coef = oracle.compute_bias_std_coef(or_n, a_bit, a_act, 5)
        x = np.linspace(0, float(a_bit.max()), 50)
        for ours, ref in ((bias_coef, g["bias_coef"]), (std_coef, g["std_coef"])):
            pa = sum(float(c) * x ** i for i, c in enumerate(ours))
            pr = sum(float(c) * x ** i for i, c in enumerate(ref))
            assert np.allclose(pa, pr, atol=1e-3), name
        if "bias_bins" not in g:
            assert not bias_coef.any() and not g["bias_coef"].any(), name


def test_counts_to_value_is_exact_scaling(oracle):
    pos = torch.tensor([0, 1, 31, 64, 2047, 2049, 20001], dtype=torch.int16)
    neg = torch.tensor([3, 0, 31, 1, 5, 2048, 7], dtype=torch.int16)
    vp, vn, vd = oracle.counts_to_value(pos, neg, 32, torch.float32)
    assert torch.equal(vp * 32, pos.float()) and torch.equal(vd * 32, (pos.int() - neg.int()).float())
    hp, hn, hd = oracle.counts_to_value(pos, neg, 32, torch.float16)
    assert hp.dtype == torch.float16 and float(hp[5]) * 32 == 2048.0  # fp16 rounds 2049 to even
