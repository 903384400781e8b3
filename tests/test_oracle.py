"""CPU tests of the oracle: it must reproduce every golden vector produced by the reference's own CPU
extensions, known-answer sums of the first configuration, and the algebraic properties of the LFSR generator."""
import os

import numpy as np
import pytest
import torch

from helpers import conv_inputs, from128, golden_cases, load_golden, quantize

PROG = (7, 8, 1)


def test_conv_golden(oracle):
    g = load_golden("sc_conv_ref_cpu.npz")
    names = golden_cases(g)
    assert len(names) >= 11
    for name in names:
        N, Cin, H, W, Cout, K, pad, stride, L, or_n, cl = (int(v) for v in g[name + "/args"])
        x, w = from128(g[name + "/x128"]), from128(g[name + "/w128"])
        if cl:
            x = x.contiguous(memory_format=torch.channels_last)
            w = w.contiguous(memory_format=torch.channels_last)
        p, n = oracle.conv2d_generic_general_split(x, w, L, -1, 16, (pad, pad), (stride, stride), PROG, or_n - 1, 1,
                                                   False, False)
        assert p.is_contiguous(memory_format=torch.channels_last) == bool(cl) or not cl
        y = (p - n).contiguous().numpy()
        assert int(y.astype(np.int64).sum()) == int(g[name + "/sum"][0]), name
        if name + "/y" in g.files:
            assert np.array_equal(y, g[name + "/y"]), name
        else:
            assert np.array_equal(y.reshape(-1)[:4096], g[name + "/y_head"]), name


def test_linear_golden(oracle):
    g = load_golden("sc_linear_ref_cpu.npz")
    for name in golden_cases(g):
        B, Cin, Cout, L, or_n = (int(v) for v in g[name + "/args"])
        x, w = from128(g[name + "/x128"]), from128(g[name + "/w128"])
        p, n = oracle.linear_generic_general(x, w, PROG, L, -1, or_n - 1, 1, False, False)
        assert np.array_equal(p.numpy(), g[name + "/pos"]), name
        assert np.array_equal(n.numpy(), g[name + "/neg"]), name


def test_fxp_golden(oracle):
    g = load_golden("fxp_conv_ref_cpu.npz")
    for name in golden_cases(g):
        N, Cin, H, W, Cout, K, pad, stride, add, p_in, p_out = (int(v) for v in g[name + "/args"])
        x, w = from128(g[name + "/x128"]), from128(g[name + "/w128"])
        y = oracle.conv2d_saturate(x, w, add, p_in, p_out, (pad, pad), (stride, stride), pad8=False)
        assert np.array_equal(y.numpy(), g[name + "/y"]), name


def test_known_answer_sums(oracle):
    """Config-1 tensors (torch CPU RNG, seed 0): sums of pos / neg for both generator variants.  The xnor=False
    rows were produced by executing the reference CPU extension; the xnor=True rows by an independent
    torch.conv2d restatement of the GPU generator."""
    torch.manual_seed(0)
    x = quantize(torch.rand(32, 3, 32, 32), 5)
    w = quantize((torch.randn(32, 3, 5, 5) * 0.1).clamp(-1, 1), 5)
    expect = {
        (32, 1, False): (19725423, 19140318), (32, 2, False): (27400328, 26533146),
        (64, 3, False): (74216246, 72961414), (32, 1, True): (25523726, 25290924),
        (32, 2, True): (39954989, 39458562), (64, 3, True): (90830324, 89499072),
    }
    for (L, or_n, xnor), (sp, sn) in expect.items():
        p, n = oracle.conv2d_generic_general_split(x, w, L, -1, 16, (2, 2), (1, 1), PROG, or_n - 1, 1, xnor, False)
        assert (int(p.long().sum()), int(n.long().sum())) == (sp, sn), (L, or_n, xnor)


@pytest.mark.parametrize("l", [3, 4, 5, 6, 7, 8])
def test_lfsr_is_maximal_length(oracle, l):
    """XOR form cycles through 1..2^l-1, XNOR form through 0..2^l-2 (all-ones is its lock-up state)."""
    for xnor, states in ((False, set(range(1, 1 << l))), (True, set(range(0, (1 << l) - 1)))):
        v = 1 - int(xnor)
        seen = set()
        for _ in range((1 << l) - 1):
            seen.add(v)
            v = oracle.lfsr_next(v, l, xnor)
        assert seen == states and v == 1 - int(xnor)
    assert oracle.lfsr_next((1 << l) - 1, l, True) == (1 << l) - 1
    assert oracle.lfsr_next(0, l, False) == 0


def test_stream_density_equals_value(oracle):
    """Over one LFSR period the comparator emits exactly `value` ones for XNOR and `value - 1` for XOR states
    (state 0 is never visited by XOR, state 2^l-1 never by XNOR)."""
    for l, L in ((5, 32), (6, 64), (7, 128)):
        for value in (0, 1, 7, L // 2, L - 1):
            bx = oracle.stream_bits(value, 3, l, True, L - 1)
            assert int(bx.sum()) == value
            bo = oracle.stream_bits(value, 3, l, False, L - 1)
            assert int(bo.sum()) == max(value - 1, 0)


@pytest.mark.parametrize("L,l", [(32, 5), (4, 3)])
def test_or_n_definition_against_torch(oracle, L, l):
    """sum_t min(count_t, n) restated with torch.conv2d on explicit bit planes.  The 4-bit case has a 3-bit LFSR
    (period 7) while values are scaled by the stream length 4 (sc_cuda.cpp:76-77, sc_cuda_kernel.cu:594-619)."""
    x, w = conv_inputs(2, 6, 7, 7, 5, 3, prec=5, seed=3)
    or_n, xnor = 2, True
    xp = torch.nn.functional.pad(x, (1, 1, 1, 1))
    aq = oracle.quantize_act(xp, L)
    wp, wn = oracle.quantize_weight(w, L)

    def planes(q, offset):
        C, H, W = q.shape[-3:]
        out = np.zeros((L,) + q.shape, dtype=np.float32)
        flat = q.reshape(-1, C * H * W)
        for b in range(flat.shape[0]):
            for i in range(C * H * W):
                seed = (offset + i) % ((1 << l) - 1) + 1 - int(xnor)
                out.reshape(L, -1, C * H * W)[:, b, i] = oracle.stream_bits(int(flat[b, i]), seed, l, xnor, L)
        return torch.from_numpy(out)

    a, bp, bn = planes(aq, 0), planes(wp, 13), planes(wn, 13)
    pos = sum(torch.nn.functional.conv2d(a[t], bp[t]).clamp(max=or_n) for t in range(L))
    neg = sum(torch.nn.functional.conv2d(a[t], bn[t]).clamp(max=or_n) for t in range(L))
    p, n = oracle.conv2d_generic_general_split(x, w, L, -1, 16, (1, 1), (1, 1), PROG, or_n - 1, 1, xnor, False)
    assert torch.equal(p, pos.to(torch.int16)) and torch.equal(n, neg.to(torch.int16))


def test_fxp_closed_form(oracle):
    """With precision_diff = 0 the sequential saturating adder equals min(sum a*w + sum (a&1)(w&1), 2^p_out)."""
    x, w = conv_inputs(2, 12, 8, 8, 6, 3, prec=7, seed=4, wscale=0.3)
    for p_in, p_out in ((5, 24), (7, 24), (7, 16)):
        y = oracle.conv2d_saturate(x, w, 0, p_in, p_out, (1, 1), (1, 1))
        a = torch.from_numpy(oracle.quantize_act(torch.nn.functional.pad(x, (1, 1, 1, 1)), 1 << p_in, "round")).double()
        wp, wn = (torch.from_numpy(t).double() for t in oracle.quantize_weight(w, 1 << p_in, "round"))
        conv = torch.nn.functional.conv2d
        pos = conv(a, wp) + conv(a % 2, wp % 2)
        neg = conv(a, wn) + conv(a % 2, wn % 2)
        cap = float(1 << max(2 * p_in, p_out))
        assert torch.equal(y.double(), pos.clamp(max=cap) - neg.clamp(max=cap)), (p_in, p_out)


def test_pointwise_reference_functions(oracle):
    s = torch.linspace(0, 6, 25, dtype=torch.float64)
    for n in (1, 2, 3, 4):
        f = oracle.orn_forward(s, n)
        e = torch.exp(-s)
        series = sum((n - i) * s ** i / float(np.prod(range(1, i + 1)) if i else 1) for i in range(n))
        assert torch.allclose(f, n - e * series, atol=1e-12)
        h = 1e-6
        num = (oracle.orn_forward(s + h, n) - oracle.orn_forward(s - h, n)) / (2 * h)
        assert torch.allclose(oracle.orn_backward(torch.ones_like(s), s, n), num, atol=1e-7)


def test_oracle_agrees_with_compiled_reference_when_present(oracle):
    """Where the reference's CPU extension is available (built by oracle/build_ref.py) run it live on a fresh
    seeded case, beyond the stored fixtures."""
    import build_ref

    mods = build_ref.load()
    if mods is None:
        pytest.skip("oracle/_ref not built (reference sources absent)")
    sc, fx = mods
    x, w = conv_inputs(2, 20, 9, 9, 12, 3, prec=6, seed=99)
    y = sc.conv2d_generic_general(x, w, 64, -1, 16, (1, 1), (2, 2), PROG, 1, 1, False, False)
    p, n = oracle.conv2d_generic_general_split(x, w, 64, -1, 16, (1, 1), (2, 2), PROG, 1, 1, False, False)
    assert torch.equal(y, p - n)
    z = fx.conv2d_saturate(x, w, 0, 6, 24, (1, 1), (1, 1))
    assert torch.equal(z, oracle.conv2d_saturate(x, w, 0, 6, 24, (1, 1), (1, 1), pad8=False))
