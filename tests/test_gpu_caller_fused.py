"""GPU tests, through the C-ABI, of the two passes that take over the caller's arithmetic on the SC conv's int16
counts: counts -> values (casts, divisions by the stream length and the pos - neg difference) and the window
statistics of the calibration fit.

counts -> values must equal the eager sequence bit for bit (every scaling is by a power of two).  The window
statistics are floating point: element counts must be equal; means and standard deviations of err agree with
the float64 oracle to 1e-5 relative + 2e-6 absolute (the kernel keeps fp32 partial sums per lane and folds them
in float64); fitted polynomials agree by value to 1e-3 at the fitted window starts."""
import numpy as np
import pytest
import torch

from helpers import golden_cases, load_golden

pytestmark = pytest.mark.gpu


def _counts(shape, hi, seed):
    g = torch.Generator().manual_seed(seed)
    return (torch.randint(0, hi + 1, shape, generator=g, dtype=torch.int32).to(torch.int16),
            torch.randint(0, hi + 1, shape, generator=g, dtype=torch.int32).to(torch.int16))


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("L,hi", [(32, 64), (64, 192), (128, 512), (32, 30000)])
def test_counts_to_value_matches_eager(ops, oracle, dtype, L, hi):
    for shape in [(1,), (7,), (8,), (4099,), (3, 16, 9, 11), (2, 64, 28, 28)]:
        pos, neg = _counts(shape, hi, L + len(shape))
        rp, rn, rd = oracle.counts_to_value(pos, neg, L, dtype)
        vp, vn, vd = ops.sc_counts_to_value(pos.cuda(), neg.cuda(), L, dtype, split=True, diff=True)
        assert vp.dtype == dtype and vp.shape == pos.shape
        assert torch.equal(vp.cpu(), rp) and torch.equal(vn.cpu(), rn) and torch.equal(vd.cpu(), rd), (shape, L)
        only = ops.sc_counts_to_value(pos.cuda(), neg.cuda(), L, dtype, split=False, diff=True)
        assert torch.equal(only.cpu(), rd)


def test_counts_to_value_layouts_and_misaligned_views(ops, oracle):
    pos, neg = _counts((2, 24, 6, 5), 64, 3)
    rp, rn, rd = oracle.counts_to_value(pos, neg, 32, torch.float16)
    p, n = pos.cuda().contiguous(memory_format=torch.channels_last), neg.cuda()  # the two signs differ in layout
    vp, vn, vd = ops.sc_counts_to_value(p, n, 32, torch.float16, diff=True)
    assert vp.stride() == p.stride()
    assert torch.equal(vp.cpu(), rp) and torch.equal(vn.cpu(), rn) and torch.equal(vd.cpu(), rd)
    flat_p, flat_n = _counts((1001,), 64, 4)
    a, b = flat_p.cuda()[1:], flat_n.cuda()[1:]                                  # 2-byte aligned starts
    vd = ops.sc_counts_to_value(a, b, 32, torch.float32, split=False, diff=True)
    assert torch.equal(vd.cpu(), oracle.counts_to_value(flat_p[1:], flat_n[1:], 32)[2])


def test_counts_to_value_rejects_bad_arguments(ops):
    pos, neg = (t.cuda() for t in _counts((16,), 10, 0))
    with pytest.raises(ValueError):
        ops.sc_counts_to_value(pos, neg, 48)                       # not a power of two
    with pytest.raises(ValueError):
        ops.sc_counts_to_value(pos.float(), neg, 32)
    with pytest.raises(ValueError):
        ops.sc_counts_to_value(pos, neg, 32, torch.bfloat16)
    with pytest.raises(RuntimeError):
        ops.sc_counts_to_value(pos.cpu(), neg.cpu(), 32)


def _windows(ops, pos, neg, vpos, vneg, L, via_half=False):
    raw = ops.sc_calib_stats(pos.cuda(), neg.cuda(), vpos.cuda(), vneg.cuda(), L, via_half).cpu()
    sums = raw[:90].view(30, 3).numpy()
    max_count = int(raw[90:].view(torch.int32)[0])
    return sums, max_count


def _check_windows(oracle, sums, max_count, pos, neg, vpos, vneg, L, tag):
    a_bit = np.concatenate([pos.numpy().reshape(-1), neg.numpy().reshape(-1)]).astype(np.float32) / L
    a_act = np.concatenate([vpos.float().numpy().reshape(-1), vneg.float().numpy().reshape(-1)])
    starts, count, mean, std = oracle.calib_windows(a_bit, a_act)
    assert max_count == int(max(pos.max(), neg.max())), tag
    assert np.array_equal(sums[:, 0].astype(np.int64), count), tag
    valid = count > 1
    cnt = sums[valid, 0]
    m = sums[valid, 1] / cnt
    s = np.sqrt(np.maximum(sums[valid, 2] - cnt * m * m, 0) / (cnt - 1))
    assert np.allclose(m, mean[valid], rtol=1e-5, atol=2e-6), tag
    assert np.allclose(s, std[valid], rtol=1e-5, atol=2e-6), tag


def _synthetic(n, L, or_n, hi, noise, seed, shape=None):
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(2):
        act = torch.rand(n, generator=g) ** 2 * hi
        cnt = torch.round((act * (1 - 0.04 * act) + noise * torch.randn(n, generator=g)) * L).clamp(0, or_n * L)
        out += [cnt.to(torch.int16), act.float()]
    pos, vpos, neg, vneg = out
    if shape is not None:
        pos, vpos, neg, vneg = (t.reshape(shape) for t in (pos, vpos, neg, vneg))
    return pos, neg, vpos, vneg


def test_calib_stats_match_reference_vectors(ops, oracle):
    npz = load_golden("calib_ref_py.npz")
    for name in golden_cases(npz):
        g = {k.split("/", 1)[1]: torch.from_numpy(npz[k]) for k in npz.files if k.startswith(name + "/")}
        L, or_n = (int(v) for v in g["args"])
        sums, max_count = _windows(ops, g["pos"], g["neg"], g["value_pos"], g["value_neg"], L)
        _check_windows(oracle, sums, max_count, g["pos"], g["neg"], g["value_pos"], g["value_neg"], L, name)
        valid = sums[:, 0] > 1
        cnt = sums[valid, 0]
        m = sums[valid, 1] / cnt
        s = np.sqrt(np.maximum(sums[valid, 2] - cnt * m * m, 0) / (cnt - 1))
        assert np.allclose(s, g["std_bins"].numpy(), rtol=1e-5, atol=2e-6), name   # the reference's own numbers
        if "bias_bins" in g:
            assert np.allclose(m, g["bias_bins"].numpy(), rtol=1e-5, atol=2e-6), name
        bias_coef, std_coef = ops.compute_bias_std_coef(or_n, g["pos"].cuda(), g["neg"].cuda(),
                                                        g["value_pos"].cuda(), g["value_neg"].cuda(), L, 5)
        # two least-squares solvers (the fixture's ran on the CPU) agree on the fitted values at the fitted points,
        # not on the coefficients of an ill-conditioned degree-5 basis nor on extrapolations beyond those points
        x = g["starts"].double().numpy()
        for ours, ref in ((bias_coef, g["bias_coef"]), (std_coef, g["std_coef"])):
            pa = sum(float(c) * x ** i for i, c in enumerate(ours.cpu()))
            pr = sum(float(c) * x ** i for i, c in enumerate(ref))
            assert np.allclose(pa, pr, atol=1e-3), name


@pytest.mark.parametrize("n,L,or_n,hi,noise,shape", [
    (1 << 20, 32, 2, 1.9, 0.05, None),
    (200_003, 64, 3, 2.8, 0.03, None),          # ragged tail, unaligned halves
    (2 * 64 * 28 * 28, 32, 2, 1.5, 0.05, (2, 64, 28, 28)),
    (5, 32, 1, 0.9, 0.05, None),
    (40_000, 128, 2, 0.2, 0.01, None),          # window spacing far below the window width
])
def test_calib_stats_match_oracle(ops, oracle, n, L, or_n, hi, noise, shape):
    pos, neg, vpos, vneg = _synthetic(n, L, or_n, hi, noise, n % 97, shape)
    sums, max_count = _windows(ops, pos, neg, vpos, vneg, L)
    _check_windows(oracle, sums, max_count, pos, neg, vpos, vneg, L, (n, L))


def test_calib_stats_edge_cases(ops, oracle):
    # all counts zero: every window is [0, 0.1)
    n = 1000
    z = torch.zeros(n, dtype=torch.int16)
    g = torch.Generator().manual_seed(1)
    v = torch.rand(n, generator=g) * 0.2
    sums, max_count = _windows(ops, z, z, v, v, 32)
    _check_windows(oracle, sums, max_count, z, z, v, v, 32, "zeros")
    assert max_count == 0 and len(set(sums[:, 0])) == 1
    # fp16 guide values, channels_last counts against contiguous guides, negative and huge guides fall in no window
    pos, neg, vpos, vneg = _synthetic(3 * 8 * 6 * 5, 32, 2, 1.9, 0.05, 7, (3, 8, 6, 5))
    vpos = vpos.clone()
    vpos.view(-1)[:4] = torch.tensor([-0.5, 1e6, float("nan"), -1e-9])
    hp, hn = vpos.half(), vneg.half()
    raw = ops.sc_calib_stats(pos.cuda().contiguous(memory_format=torch.channels_last), neg.cuda(), hp.cuda(),
                             hn.cuda(), 32).cpu()
    sums = raw[:90].view(30, 3).numpy()
    _check_windows(oracle, sums, int(raw[90:].view(torch.int32)[0]), pos, neg, hp, hn, 32, "half")
    # the same call twice gives the same block (the block is cleared by the call)
    a = ops.sc_calib_stats(pos.cuda(), neg.cuda(), vpos.cuda(), vneg.cuda(), 32)
    b = ops.sc_calib_stats(pos.cuda(), neg.cuda(), vpos.cuda(), vneg.cuda(), 32)
    assert torch.equal(a[:90].cpu().view(30, 3)[:, 0], b[:90].cpu().view(30, 3)[:, 0])
    # empty input
    e16, e32 = torch.zeros(0, dtype=torch.int16).cuda(), torch.zeros(0).cuda()
    assert not ops.sc_calib_stats(e16, e16, e32, e32, 32)[:90].any()


def test_calib_two_stage_calls_equal_single_call(ops, oracle):
    """rexsc_sc_calib_max + rexsc_sc_calib_windows == rexsc_sc_calib_stats; a maximum raised between the stages (what
    an all-reduce over ranks does on a shard that does not hold the global maximum) moves the windows accordingly."""
    pos, neg, vpos, vneg = _synthetic(50_000, 32, 2, 1.9, 0.05, 3)
    args = (pos.cuda(), neg.cuda(), vpos.cuda(), vneg.cuda(), 32)
    one = ops.sc_calib_stats(*args).cpu()
    seen = []
    two = ops.sc_calib_stats(*args, between=lambda st: seen.append(int(st[90:].view(torch.int32)[0]))).cpu()
    assert seen == [int(max(pos.max(), neg.max()))]
    # sums are folded with double atomics whose order varies from launch to launch: equal to rounding, counts exactly
    assert torch.equal(one[90:], two[90:]) and torch.equal(one[:90].view(30, 3)[:, 0], two[:90].view(30, 3)[:, 0])
    assert torch.allclose(one[:90], two[:90], rtol=1e-10, atol=1e-9)

    def raise_max(st):
        st[90:].view(torch.int32)[0] = 80
    moved = ops.sc_calib_stats(*args, between=raise_max).cpu()
    a_bit = np.concatenate([pos.numpy(), neg.numpy()]).astype(np.float32) / 32
    a_act = np.concatenate([vpos.numpy(), vneg.numpy()])
    ref = oracle.calib_window_sums(a_bit, a_act, top=80 / 32)
    got = moved[:90].view(30, 3).numpy()
    assert np.array_equal(got[:, 0], ref[:, 0])
    assert np.allclose(got[:, 1:], ref[:, 1:], rtol=1e-5, atol=1e-4)
    # single-process job: across_ranks is a no-op and gives the same fit
    b0, s0 = ops.compute_bias_std_coef(2, *args, 5)
    b1, s1 = ops.compute_bias_std_coef(2, *args, 5, across_ranks=True)
    assert torch.allclose(b0, b1, rtol=1e-3, atol=1e-5) and torch.allclose(s0, s1, rtol=1e-3, atol=1e-5)


@pytest.mark.parametrize("L,max_count", [(32, 64), (32, 37), (128, 1), (128, 2), (128, 4), (4096, 3), (64, 192)])
def test_calib_guides_on_and_next_to_window_edges(ops, oracle, L, max_count):
    """Guide values exactly on every window start and end, and one fp32 step below and above each: membership must
    follow the exact fp32 comparisons of the reference, whatever the kernel's estimate of the window index says."""
    top = max_count / L
    starts = np.linspace(0, top, 30)
    edges = np.concatenate([starts.astype(np.float32), (starts + 0.1).astype(np.float32)])
    vals = np.concatenate([edges, np.nextafter(edges, np.float32(-np.inf)), np.nextafter(edges, np.float32(np.inf)),
                           (edges[:-1] + edges[1:]) / 2]).astype(np.float32)
    n = vals.size
    g = torch.Generator().manual_seed(L + max_count)
    pos = torch.randint(0, max_count + 1, (n,), generator=g, dtype=torch.int32).to(torch.int16)
    neg = torch.randint(0, max_count + 1, (n,), generator=g, dtype=torch.int32).to(torch.int16)
    pos[0] = max_count
    vpos = torch.from_numpy(vals)
    vneg = torch.from_numpy(vals[::-1].copy())
    sums, got_max = _windows(ops, pos, neg, vpos, vneg, L)
    _check_windows(oracle, sums, got_max, pos, neg, vpos, vneg, L, (L, max_count))
