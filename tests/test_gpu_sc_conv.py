"""GPU parity of the SC conv2d / linear forward (through the C-ABI) against the CPU oracle and against the
golden vectors produced by the reference's own CPU extension.  Bit-exact: integer work."""
import numpy as np
import pytest
import torch

from helpers import conv_inputs, from128, golden_cases, load_golden

pytestmark = pytest.mark.gpu

PROG = (7, 8, 1)


def run_ours(ops, x, w, L, pad, stride, or_n, xnor, kernel="auto", gen=1, prog=PROG, lfsr=-1, dtype=None):
    ops.set_conv_kernel(kernel)
    try:
        xd, wd = x.cuda(), w.cuda()
        if dtype is not None:
            xd, wd = xd.to(dtype), wd.to(dtype)
        if x.is_contiguous(memory_format=torch.channels_last) and not x.is_contiguous():
            xd = xd.contiguous(memory_format=torch.channels_last)
        if w.is_contiguous(memory_format=torch.channels_last) and not w.is_contiguous():
            wd = wd.contiguous(memory_format=torch.channels_last)
        p, n = ops.conv2d_generic_general_split_acc(xd, wd, L, lfsr, 16, (pad, pad), (stride, stride), prog,
                                                    or_n - 1, gen, xnor, False)
        assert ops.workspace_status() == 0
        return p, n
    finally:
        ops.set_conv_kernel("auto")


def assert_same(ours, ref, what):
    p, n = ours
    rp, rn = ref
    assert p.dtype == torch.int16 and n.dtype == torch.int16
    assert p.shape == rp.shape
    # same memory format (strides of size-1 dimensions are arbitrary, so compare the format predicates)
    for fmt in (torch.contiguous_format, torch.channels_last):
        assert p.is_contiguous(memory_format=fmt) == rp.is_contiguous(memory_format=fmt), f"{what}: memory format"
    assert torch.equal(p.cpu(), rp), f"{what}: pos differs ({(p.cpu() != rp).sum().item()} elements)"
    assert torch.equal(n.cpu(), rn), f"{what}: neg differs ({(n.cpu() != rn).sum().item()} elements)"


def _run_or_skip_unsupported(fn, kernel):
    """Forcing a kernel on a shape it does not cover is refused with REXSC_E_UNSUPPORTED (ValueError)."""
    try:
        return fn()
    except ValueError as exc:
        if kernel in ("tiled", "tensor") and "UNSUPPORTED" in str(exc):
            return None
        raise


@pytest.mark.parametrize("kernel", ["direct", "tiled", "tensor"])
def test_golden_reference_cpu_vectors(ops, kernel):
    """xnor=False: pos - neg must equal what the reference's CPU extension returned."""
    g = load_golden("sc_conv_ref_cpu.npz")
    for name in golden_cases(g):
        N, Cin, H, W, Cout, K, pad, stride, L, or_n, cl = (int(v) for v in g[name + "/args"])
        if kernel == "tiled" and or_n > 4:
            continue  # plain-count / large-n accumulation is not in the ALU tiled kernel
        x, w = from128(g[name + "/x128"]), from128(g[name + "/w128"])
        if cl:
            x = x.contiguous(memory_format=torch.channels_last)
            w = w.contiguous(memory_format=torch.channels_last)
        res = _run_or_skip_unsupported(lambda: run_ours(ops, x, w, L, pad, stride, or_n, False, kernel), kernel)
        if res is None:
            assert kernel == "tensor" and K > 3   # only filters larger than 3x3 are outside the tensor kernel
            continue
        p, n = res
        y = (p - n).contiguous().cpu().numpy()
        assert int(y.astype(np.int64).sum()) == int(g[name + "/sum"][0]), name
        if name + "/y" in g.files:
            assert np.array_equal(y, g[name + "/y"]), name
        else:
            assert np.array_equal(y.reshape(-1)[:4096], g[name + "/y_head"]), name


CASES = [
    # N, Cin, H, W, Cout, K, pad, stride, L, or_n, channels_last
    (2, 3, 12, 12, 8, 5, 2, 1, 32, 1, False),
    (2, 32, 10, 10, 16, 3, 1, 1, 32, 2, True),
    (3, 64, 9, 9, 70, 3, 1, 1, 32, 2, True),      # Cout not a multiple of 32
    (2, 70, 9, 9, 40, 3, 1, 2, 32, 2, False),     # stride 2, Cin not a multiple of 8
    (3, 64, 8, 8, 24, 1, 0, 2, 64, 3, True),      # 1x1 stride 2, two word planes
    (2, 16, 4, 4, 10, 4, 0, 1, 128, 1, False),    # 4x4 -> 1x1 output, four word planes
    (1, 5, 12, 7, 7, 5, 2, 1, 32, 4, False),      # non-square, OR-4
    (5, 24, 7, 7, 33, 3, 1, 1, 32, 3, True),      # tile spans several images
    (2, 8, 6, 6, 5, 3, 1, 1, 16, 1, False),       # L < 32
    (1, 130, 5, 5, 4, 3, 1, 1, 32, 2, False),     # many channel chunks, tiny tile
    (2, 16, 20, 20, 12, 7, 3, 2, 32, 2, True),    # 7x7 stride 2
]


@pytest.mark.parametrize("xnor", [False, True])
@pytest.mark.parametrize("kernel", ["direct", "tiled", "tensor"])
@pytest.mark.parametrize("case", CASES)
def test_parity_vs_oracle(ops, oracle, case, kernel, xnor):
    N, Cin, H, W, Cout, K, pad, stride, L, or_n, cl = case
    if kernel == "tensor" and K > 3:
        pytest.skip("the tensor-core kernel stages at most 9 filter taps")
    x, w = conv_inputs(N, Cin, H, W, Cout, K, prec=7, seed=hash(case) % 1000)
    if cl:
        x = x.contiguous(memory_format=torch.channels_last)
        w = w.contiguous(memory_format=torch.channels_last)
    ref = oracle.conv2d_generic_general_split(x, w, L, -1, 16, (pad, pad), (stride, stride), PROG, or_n - 1, 1,
                                              xnor, False)
    ours = run_ours(ops, x, w, L, pad, stride, or_n, xnor, kernel)
    assert_same(ours, ref, f"{case} {kernel} xnor={xnor}")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_half_precision_inputs(ops, oracle, dtype):
    x, w = conv_inputs(2, 16, 9, 9, 12, 3, prec=5, seed=11)
    xq, wq = x.to(dtype).float(), w.to(dtype).float()
    ref = oracle.conv2d_generic_general_split(xq, wq, 32, -1, 16, (1, 1), (1, 1), PROG, 1, 1, True, False)
    ours = run_ours(ops, x, w, 32, 1, 1, 2, True, "auto", dtype=dtype)
    assert_same(ours, ref, str(dtype))


def test_mixed_layouts(ops, oracle):
    """channels_last activation with OIHW weight and the reverse: layout only changes addressing."""
    x, w = conv_inputs(2, 16, 8, 8, 8, 3, seed=5)
    ref = oracle.conv2d_generic_general_split(x, w, 32, -1, 16, (1, 1), (1, 1), PROG, 1, 1, True, False)
    xc = x.contiguous(memory_format=torch.channels_last)
    wc = w.contiguous(memory_format=torch.channels_last)
    p, n = run_ours(ops, xc, w, 32, 1, 1, 2, True)
    assert torch.equal(p.cpu().contiguous(), ref[0]) and torch.equal(n.cpu().contiguous(), ref[1])
    assert p.is_contiguous(memory_format=torch.channels_last)
    p, n = run_ours(ops, x, wc, 32, 1, 1, 2, True)
    assert torch.equal(p.cpu(), ref[0]) and torch.equal(n.cpu(), ref[1])
    assert p.is_contiguous()


def test_combined_output_op(ops, oracle):
    x, w = conv_inputs(2, 8, 8, 8, 8, 3, seed=6)
    ref = oracle.conv2d_generic_general_split(x, w, 32, -1, 16, (1, 1), (1, 1), PROG, 0, 1, True, False)
    y = ops.conv2d_generic_general_acc(x.cuda(), w.cuda(), 32, -1, 16, (1, 1), (1, 1), PROG, 0, 1, True, False)
    assert y.dtype == torch.int16 and torch.equal(y.cpu(), ref[0] - ref[1])


@pytest.mark.parametrize("kernel", ["auto", "tensor"])
@pytest.mark.parametrize("or_n", [7, 51201])
def test_large_n_and_plain_count(ops, oracle, or_n, kernel):
    x, w = conv_inputs(1, 40, 6, 6, 9, 3, prec=5, seed=7)
    ref = oracle.conv2d_generic_general_split(x, w, 32, -1, 16, (1, 1), (1, 1), PROG, or_n - 1, 1, True, False)
    ours = run_ours(ops, x, w, 32, 1, 1, or_n, True, kernel)
    assert_same(ours, ref, f"or_n={or_n} {kernel}")


def test_generator_options(ops, oracle):
    """AND-2 generator replication, progressive loading and an explicit lfsr_length."""
    x, w = conv_inputs(2, 12, 7, 7, 6, 3, seed=8)
    for gen, prog, lfsr, L in [(2, PROG, -1, 32), (1, (7, 2, 4), -1, 32), (1, PROG, 7, 32), (3, (7, 3, 2), -1, 16)]:
        for xnor in (False, True):
            ref = oracle.conv2d_generic_general_split(x, w, L, lfsr, 16, (1, 1), (1, 1), prog, 1, gen, xnor, False)
            for kernel in ("direct", "tiled", "tensor"):
                ours = run_ours(ops, x, w, L, 1, 1, 2, xnor, kernel, gen=gen, prog=prog, lfsr=lfsr)
                assert_same(ours, ref, f"gen={gen} prog={prog} lfsr={lfsr} {kernel} xnor={xnor}")


def test_short_streams_scale_by_the_stream_length(ops, oracle):
    """bit_length 2 and 4 with a derived LFSR length: the LFSR has 3 bits (sc_cuda_kernel.cu:594-619 falls through)
    but values are scaled by bit_length itself, not by 2^3 (sc_cuda.cpp:76-77,90-91)."""
    x, w = conv_inputs(2, 40, 7, 7, 9, 3, seed=21, wscale=0.6)
    for L in (2, 4):
        for xnor in (False, True):
            ref = oracle.conv2d_generic_general_split(x, w, L, -1, 16, (1, 1), (1, 1), PROG, 1, 1, xnor, False)
            assert L == 2 or int(ref[0].sum()) > 0
            for kernel in ("direct", "tiled", "tensor"):
                assert_same(run_ours(ops, x, w, L, 1, 1, 2, xnor, kernel), ref, f"L={L} {kernel} xnor={xnor}")
        # with the LFSR length given, the scale is 2^lfsr_length instead
        ref = oracle.conv2d_generic_general_split(x, w, L, 3, 16, (1, 1), (1, 1), PROG, 1, 1, True, False)
        assert_same(run_ours(ops, x, w, L, 1, 1, 2, True, "auto", lfsr=3), ref, f"L={L} lfsr=3")


def test_asymmetric_padding_and_stride(ops, oracle):
    x, w = conv_inputs(2, 8, 9, 11, 6, 3, seed=9)
    ref = oracle.conv2d_generic_general_split(x, w, 32, -1, 16, (2, 1), (2, 1), PROG, 1, 1, True, False)
    p, n = ops.conv2d_generic_general_split_acc(x.cuda(), w.cuda(), 32, -1, 16, (2, 1), (2, 1), PROG, 1, 1, True,
                                                False)
    assert torch.equal(p.cpu(), ref[0]) and torch.equal(n.cpu(), ref[1])


def test_edge_values(ops, oracle):
    """0, 1-eps, 1, >1 and negative activations; weights at +-1 and 0 (quantiser clamps, zero streams)."""
    x = torch.tensor([0.0, 1 / 128, 0.5, 1 - 1 / 128, 1.0, 1.5, -0.25, 31 / 32]).repeat(8 * 8 * 2)[:8 * 8 * 8]
    x = x.reshape(1, 8, 8, 8).contiguous()
    w = torch.tensor([0.0, 1.0, -1.0, 1 / 128, -1 / 128, 0.5, -0.5, 0.999]).repeat(4 * 8 * 9)[:4 * 8 * 9]
    w = w.reshape(4, 8, 3, 3).contiguous()
    for xnor in (False, True):
        ref = oracle.conv2d_generic_general_split(x, w, 32, -1, 16, (1, 1), (1, 1), PROG, 1, 1, xnor, False)
        assert_same(run_ours(ops, x, w, 32, 1, 1, 2, xnor), ref, f"edge xnor={xnor}")


def test_linear_golden_and_oracle(ops, oracle):
    g = load_golden("sc_linear_ref_cpu.npz")
    for name in golden_cases(g):
        B, Cin, Cout, L, or_n = (int(v) for v in g[name + "/args"])
        x, w = from128(g[name + "/x128"]), from128(g[name + "/w128"])
        p, n = ops.linear_generic_general_acc(x.cuda(), w.cuda(), PROG, L, -1, or_n - 1, 1, True, False)
        assert np.array_equal(p.cpu().numpy(), g[name + "/pos"]), name
        assert np.array_equal(n.cpu().numpy(), g[name + "/neg"]), name
    # ragged sizes only the oracle covers
    gen = torch.Generator().manual_seed(3)
    x = torch.rand(37, 45, generator=gen)
    w = (torch.randn(19, 45, generator=gen) * 0.2).clamp(-1, 1)
    rp, rn = oracle.linear_generic_general(x, w, PROG, 64, -1, 2, 1, True, False)
    p, n = ops.linear_generic_general_acc(x.cuda(), w.cuda(), PROG, 64, -1, 2, 1, True, False)
    assert torch.equal(p.cpu(), rp) and torch.equal(n.cpu(), rn)


def _torch_loop_linear_counts(x, w, L, seeds, or1):
    """numpy restatement of the per-bit loop of the reference's linear_generic with generator='lfsr' and shared
    generators (utils_functional.py:147-165 seeds, :254-271 LFSR per stream length, :1016-1036 loop): returns the
    counts sum_t OR_c(a_t & w_t) (or the plain sums) per sign."""
    l = {8: 3, 16: 4, 32: 5, 64: 6, 128: 7}[L]
    taps = {3: (2, 1), 4: (3, 2), 5: (4, 2), 6: (5, 4), 7: (6, 5)}[l]
    step = lambda v: (((v >> taps[0]) ^ (v >> taps[1])) & 1) | ((v << 1) & ((1 << l) - 1))
    c = np.arange(x.shape[1])
    ra, rp, rn = c % (L - 1) + 1, (c + seeds[0]) % (L - 1) + 1, (c + seeds[1]) % (L - 1) + 1
    xa = x.astype(np.float64) * L
    wp, wn = np.clip(w.astype(np.float64) * L, 0, None), np.clip(-w.astype(np.float64) * L, 0, None)
    pos = np.zeros((x.shape[0], w.shape[0]), np.int64)
    neg = np.zeros_like(pos)
    for _ in range(L):
        ra, rp, rn = step(ra), step(rp), step(rn)
        a = (xa > ra).astype(np.int64)
        sp, sn = a @ (wp > rp).astype(np.int64).T, a @ (wn > rn).astype(np.int64).T
        pos += np.minimum(sp, 1) if or1 else sp
        neg += np.minimum(sn, 1) if or1 else sn
    return pos, neg


@pytest.mark.parametrize("kernel", ["direct", "tiled", "tensor"])
def test_linear_with_weight_seed_offsets(ops, kernel):
    """rexsc_sc_linear_fwd_seeded on all three kernels: seed offsets (67, 37) give the counts of the front end's torch
    bit loop (restated above), other offsets differ from the extension's (13, 13), negative offsets are refused."""
    gen = torch.Generator().manual_seed(17)
    for L, B, Cin, Cout in ((32, 9, 70, 33), (128, 5, 64, 64)):
        top = (L - 1) / L
        x = ((torch.rand(B, Cin, generator=gen) * 128).floor() / 128).clamp(max=top)
        w = torch.randn(Cout, Cin, generator=gen) * 0.08
        w[:, ::5] *= 6
        w = ((w.clamp(-1, 1) * 128).round() / 128).clamp(-top, top)
        for or_n in (1, 51201):
            rp, rn = _torch_loop_linear_counts(x.numpy(), w.numpy(), L, (67, 37), or_n == 1)
            ops.set_conv_kernel(kernel)
            try:
                p, n = ops.linear_generic_general_acc(x.cuda(), w.cuda(), PROG, L, -1, or_n - 1, 1, False, False,
                                                      weight_seeds=(67, 37))
                d, _ = ops.linear_generic_general_acc(x.cuda(), w.cuda(), PROG, L, -1, or_n - 1, 1, False, False)
            except ValueError as exc:
                assert kernel != "direct" and "UNSUPPORTED" in str(exc)
                continue
            finally:
                ops.set_conv_kernel("auto")
            assert np.array_equal(p.cpu().numpy(), rp) and np.array_equal(n.cpu().numpy(), rn), (kernel, L, or_n)
            assert not torch.equal(p, d)
    with pytest.raises(ValueError):
        ops.linear_generic_general_acc(x.cuda(), w.cuda(), PROG, 32, -1, 0, 1, False, False, weight_seeds=(-1, 13))


def test_lut_matches_oracle_streams(ops, oracle):
    for l, L, xnor in [(5, 32, True), (5, 32, False), (6, 64, True), (7, 128, False), (3, 8, True)]:
        lut = ops.build_lfsr_lut(l, L, 1, xnor).cpu().numpy().astype(np.uint32)
        period = (1 << l) - 1
        for phase in (0, 1, period // 2, period - 1):
            for value in (0, 1, (1 << l) // 2, (1 << l) - 1):
                bits = oracle.stream_bits(value, phase + 1 - int(xnor), l, xnor, L)
                words = np.zeros(lut.shape[2], dtype=np.uint32)
                for t, b in enumerate(bits):
                    if b:
                        words[t // 32] |= np.uint32(1 << (t % 32))
                assert np.array_equal(lut[phase, value], words), (l, L, xnor, phase, value)


def test_rejects_bad_arguments(ops):
    x = torch.rand(1, 4, 6, 6).cuda()
    w = torch.rand(4, 4, 3, 3).cuda()
    with pytest.raises(ValueError):
        ops.conv2d_generic_general_split_acc(x, w, 48, -1, 16, (0, 0), (1, 1), PROG, 0, 1, True, False)  # L not 2^k
    with pytest.raises(ValueError):
        ops.conv2d_generic_general_split_acc(x, w, 32, -1, 16, (0, 0), (1, 1), PROG, -2, 1, True, False)
    with pytest.raises(RuntimeError):
        ops.conv2d_generic_general_split_acc(x.cpu(), w.cpu(), 32, -1, 16, (0, 0), (1, 1), PROG, 0, 1, True, False)


def test_full_size_properties(ops):
    """ResNet-18 layer-1 shape at batch 32 (too large for the oracle): direct == tiled, determinism, bounds,
    zero weights give zero, and a batch permutation permutes the output (samples are independent)."""
    g = torch.Generator().manual_seed(1)
    x = torch.rand(32, 64, 56, 56, generator=g).cuda().contiguous(memory_format=torch.channels_last)
    w = (torch.randn(64, 64, 3, 3, generator=g) * 0.05).clamp(-1, 1).cuda().contiguous(
        memory_format=torch.channels_last)
    args = (32, -1, 16, (1, 1), (1, 1), PROG, 1, 1, True, False)
    ops.set_conv_kernel("tiled")
    p1, n1 = ops.conv2d_generic_general_split_acc(x, w, *args)
    p2, n2 = ops.conv2d_generic_general_split_acc(x, w, *args)
    ops.set_conv_kernel("direct")
    p3, n3 = ops.conv2d_generic_general_split_acc(x, w, *args)
    ops.set_conv_kernel("tensor")
    p4, n4 = ops.conv2d_generic_general_split_acc(x, w, *args)
    ops.set_conv_kernel("auto")
    assert ops.workspace_status() == 0
    assert torch.equal(p1, p2) and torch.equal(n1, n2)
    assert torch.equal(p1, p3) and torch.equal(n1, n3)
    assert torch.equal(p1, p4) and torch.equal(n1, n4)
    assert int(p1.min()) >= 0 and int(p1.max()) <= 64 and int(n1.min()) >= 0 and int(n1.max()) <= 64
    pz, nz = ops.conv2d_generic_general_split_acc(x, torch.zeros_like(w), *args)
    assert int(pz.abs().max()) == 0 and int(nz.abs().max()) == 0
    perm = torch.randperm(32, generator=g).cuda()
    pp, _ = ops.conv2d_generic_general_split_acc(x[perm].contiguous(memory_format=torch.channels_last), w, *args)
    assert torch.equal(pp, p1[perm])
    # negating the weights swaps the two outputs
    ps, ns = ops.conv2d_generic_general_split_acc(x, -w, *args)
    assert torch.equal(ps, n1) and torch.equal(ns, p1)


def test_randomised_shapes_tiled_and_direct_vs_oracle(ops, oracle):
    """40 seeded random configurations (shape, stride, padding, stream length, OR-n, layout, generator)."""
    import random

    rng = random.Random(20241)
    for trial in range(40):
        K = rng.choice([1, 1, 3, 3, 3, 5])
        KW = K if rng.random() < 0.8 else rng.choice([1, 2, 3])
        stride = rng.choice([1, 1, 2, 3])
        pad = rng.choice([0, 1, 2]) if K > 1 else 0
        H = rng.randint(max(K, 3), 14)
        W = rng.randint(max(KW, 3), 14)
        N = rng.randint(1, 5)
        Cin = rng.choice([1, 3, 8, 9, 16, 31, 40])
        Cout = rng.choice([1, 5, 32, 33, 48])
        L = rng.choice([8, 16, 32, 32, 64, 128])
        or_n = rng.choice([1, 2, 2, 3, 4])
        cl = rng.random() < 0.5
        xnor = rng.random() < 0.6
        if H + 2 * pad < K or W + 2 * pad < KW:
            continue
        x, w = conv_inputs(N, Cin, H, W, Cout, K, prec=7, seed=trial, KW=KW)
        if cl:
            x = x.contiguous(memory_format=torch.channels_last)
            w = w.contiguous(memory_format=torch.channels_last)
        ref = oracle.conv2d_generic_general_split(x, w, L, -1, 16, (pad, pad), (stride, stride), PROG, or_n - 1, 1,
                                                  xnor, False)
        for kernel in ("tiled", "tensor", "direct"):
            ours = _run_or_skip_unsupported(lambda: run_ours(ops, x, w, L, pad, stride, or_n, xnor, kernel), kernel)
            if ours is None:
                continue  # shape outside that kernel: the direct kernel covers it
            assert_same(ours, ref, f"trial {trial}: {(N, Cin, H, W, Cout, K, KW, pad, stride, L, or_n, cl, xnor)} {kernel}")


TENSOR_CASES = [
    # N, Cin, H, W, Cout, K, pad, stride, L, or_n, channels_last -- shapes that exercise the tensor-core kernel's
    # variants: residue planes of strided layers (32-channel steps, several patch rows per thread), odd channel-word
    # counts (a last chunk with one word), several 64-channel output chunks, tiles that span images, long streams
    # (per-slot descaling) and plain counting
    (5, 64, 56, 56, 128, 3, 1, 2, 32, 2, True),    # ResNet stride-2 3x3: 4 residue planes
    (3, 96, 17, 15, 70, 3, 1, 2, 32, 2, True),     # 3 channel words, ragged Cout, non-square, stride 2
    (2, 160, 12, 12, 130, 3, 1, 1, 32, 2, True),   # 5 channel words: chunks of 2, 2, 1; three output chunks
    (2, 64, 12, 12, 64, 2, 0, 2, 32, 2, True),     # 2x2 stride 2
    (4, 64, 14, 14, 64, 1, 0, 2, 32, 2, True),     # 1x1 stride 2: stored grid keeps residue 0 only
    (2, 40, 11, 13, 30, 3, 1, 1, 128, 3, False),   # NCHW, L=128: running sums descaled every slot
    (2, 64, 9, 9, 64, 3, 1, 1, 64, 4, True),       # two word planes, OR-4
    (70, 32, 4, 4, 8, 3, 1, 1, 32, 1, False),      # tiles span many small images
    (2, 64, 10, 10, 32, 3, 1, 3, 32, 2, True),     # stride 3: 9 residue planes
]


@pytest.mark.parametrize("case", TENSOR_CASES)
def test_tensor_kernel_variants_vs_direct(ops, case):
    """The tensor-core kernel against the direct kernel (itself pinned to the oracle above) on shapes too large for
    the oracle; both receive the same inputs through the public op."""
    N, Cin, H, W, Cout, K, pad, stride, L, or_n, cl = case
    x, w = conv_inputs(N, Cin, H, W, Cout, K, prec=7, seed=hash(case) % 1000)
    if cl:
        x = x.contiguous(memory_format=torch.channels_last)
        w = w.contiguous(memory_format=torch.channels_last)
    ref = run_ours(ops, x, w, L, pad, stride, or_n, True, "direct")
    got = _run_or_skip_unsupported(lambda: run_ours(ops, x, w, L, pad, stride, or_n, True, "tensor"), "tensor")
    if got is None:
        assert stride == 3, f"{case}: only the 9-plane stride-3 case may be outside the tensor kernel"
        return
    assert torch.equal(got[0], ref[0]) and torch.equal(got[1], ref[1]), str(case)
    plain = run_ours(ops, x, w, L, pad, stride, 51201, True, "tensor")   # plain counting (n above any count)
    plain_ref = run_ours(ops, x, w, L, pad, stride, 51201, True, "direct")
    assert torch.equal(plain[0], plain_ref[0]) and torch.equal(plain[1], plain_ref[1]), f"{case} plain count"


COMPACT_CASES = [
    # N, Cin, H, W, Cout, L, or_n, channels_last, dtype -- 3x3 stride-1 layers of the tensor-core kernel, whose
    # activation grid drops the shared zero border (one row and one column per image instead of two)
    (6, 64, 7, 7, 64, 32, 2, True, torch.float32),      # few tiles: time slots split over CTAs, atomically added
    (37, 64, 7, 9, 128, 32, 2, True, torch.float16),    # tiles span images; half-precision staging
    (3, 96, 14, 14, 70, 64, 3, True, torch.float32),    # two word planes, ragged output channels
    (5, 64, 8, 8, 64, 32, 1, False, torch.float32),     # NCHW fp32: single-launch expand with 4-byte staging
    (5, 40, 8, 6, 64, 32, 2, False, torch.float16),     # NCHW fp16: single-launch expand staged through registers
    (300, 32, 4, 4, 64, 32, 2, True, torch.float32),    # more tiles than SMs
]


@pytest.mark.parametrize("case", COMPACT_CASES)
def test_compact_grid_of_3x3_layers(ops, case):
    """The same layer three ways through the tensor-core kernel, each against the direct kernel (pinned to the oracle
    above): padding done by the op (compact grid by construction), padding done by the caller as the reference's
    front end does (border checked on the device, compact grid), and caller-padded data whose border is NOT zero in
    one place (the check fails, the standard grid is used)."""
    N, Cin, H, W, Cout, L, or_n, cl, dtype = case
    x, w = conv_inputs(N, Cin, H, W, Cout, 3, prec=7, seed=sum(case[:7]))
    fmt = torch.channels_last if cl else torch.contiguous_format
    x = x.to(dtype).contiguous(memory_format=fmt)
    w = w.to(dtype).contiguous(memory_format=fmt)
    ref = run_ours(ops, x, w, L, 1, 1, or_n, True, "direct")
    got = run_ours(ops, x, w, L, 1, 1, or_n, True, "tensor")
    assert torch.equal(got[0], ref[0]) and torch.equal(got[1], ref[1]), f"{case}: op-padded"

    xp = torch.nn.functional.pad(x, (1, 1, 1, 1)).contiguous(memory_format=fmt)
    got = run_ours(ops, xp, w, L, 0, 1, or_n, True, "tensor")
    assert torch.equal(got[0], ref[0]) and torch.equal(got[1], ref[1]), f"{case}: caller-padded"
    # values that quantise to zero are as good as zeros
    xn = xp.clone()
    xn[:, :, 0, :] = -0.5
    xn[:, :, :, -1] = float("nan")
    got = run_ours(ops, xn, w, L, 0, 1, or_n, True, "tensor")
    assert torch.equal(got[0], ref[0]) and torch.equal(got[1], ref[1]), f"{case}: negative / NaN border"

    for where in ((N - 1, Cin - 1, H + 1, W + 1), (0, 0, 0, 3), (N // 2, 1, 2, 0)):
        xb = xp.clone()
        xb[where] = 0.75
        ref_b = run_ours(ops, xb, w, L, 0, 1, or_n, True, "direct")
        got = run_ours(ops, xb, w, L, 0, 1, or_n, True, "tensor")
        assert torch.equal(got[0], ref_b[0]) and torch.equal(got[1], ref_b[1]), f"{case}: live border at {where}"
    # and the next call on a clean border takes the compact grid again
    got = run_ours(ops, xp, w, L, 0, 1, or_n, True, "tensor")
    assert torch.equal(got[0], ref[0]) and torch.equal(got[1], ref[1]), f"{case}: caller-padded, after a fallback"


def test_compact_grid_with_prepared_weights(ops):
    """Weights expanded once, caller-padded activations per call (their border decides the grid on every call)."""
    g = torch.Generator().manual_seed(11)
    w = (torch.randn(64, 64, 3, 3, generator=g) * 0.1).clamp(-1, 1).cuda().contiguous(memory_format=torch.channels_last)
    args = (32, -1, (0, 0), (1, 1), PROG, 1, 1, True)
    xs = []
    for i in range(4):
        x = torch.nn.functional.pad(torch.rand(9, 64, 7, 7, generator=g), (1, 1, 1, 1))
        if i % 2:
            x[3, 5, 8, 2] = 0.5
        xs.append(x.cuda().contiguous(memory_format=torch.channels_last))
    conv = ops.PreparedConv(w, xs[0].shape, xs[0].dtype, True, *args)
    for x in xs:
        pos, neg = conv(x)
        ops.set_conv_kernel("direct")
        try:
            rpos, rneg = ops.conv2d_generic_general_split_acc(x, w, 32, -1, 16, (0, 0), (1, 1), PROG, 1, 1, True, False)
        finally:
            ops.set_conv_kernel("auto")
        assert torch.equal(pos, rpos) and torch.equal(neg, rneg)


def test_kernel_launch_counter(ops):
    """rexsc_kernel_launch_count counts this library's kernels: a tensor-core conv whose padding the op does takes the
    single-launch expand stage and the conv kernel, plus one clearing kernel when CTAs share tiles; the ALU path takes
    tables, two expansions and the accumulate kernel."""
    from rexsc_b200 import _lib
    lib = _lib.load()
    x, w = conv_inputs(4, 64, 8, 8, 64, 3, prec=7, seed=3)
    x = x.cuda().contiguous(memory_format=torch.channels_last)
    w = w.cuda().contiguous(memory_format=torch.channels_last)

    def launches(kernel, pad, xin):
        ops.set_conv_kernel(kernel)
        try:
            c0 = lib.rexsc_kernel_launch_count()
            ops.conv2d_generic_general_split_acc(xin, w, 32, -1, 16, (pad, pad), (1, 1), PROG, 1, 1, True, False)
            return lib.rexsc_kernel_launch_count() - c0
        finally:
            ops.set_conv_kernel("auto")

    assert launches("tensor", 1, x) in (2, 3)
    assert launches("direct", 1, x) == 4
    # caller-padded: border check inside the expand launch, the gated standard-grid expand and conv behind it
    xp = torch.nn.functional.pad(x, (1, 1, 1, 1)).contiguous(memory_format=torch.channels_last)
    assert launches("tensor", 0, xp) in (4, 5)


def test_auto_kernel_choice(ops):
    """AUTO resolves to the tensor-core kernel for every layer shape of the bench workload that has >= 32 input
    channels and at most 9 taps, and to an ALU kernel for thin inputs and large filters."""
    import ctypes as C
    from rexsc_b200 import _lib
    lib = _lib.load()

    def choice(N, Cin, H, Cout, K, stride):
        d = _lib.ScConvDesc()
        d.batch, d.c_in, d.h_in, d.w_in, d.c_out, d.kh, d.kw = N, Cin, H, H, Cout, K, K
        d.stride_h = d.stride_w = stride
        d.act_channels_last = d.w_channels_last = d.out_channels_last = 1
        d.bit_length, d.lfsr_length, d.bin_config, d.gen_config, d.xnor = 32, -1, 1, 1, 1
        d.prog_total_width, d.prog_load_width, d.prog_load_wait = PROG
        return lib.rexsc_sc_conv2d_kernel_choice(C.byref(d))

    assert choice(256, 64, 58, 64, 3, 1) == 3
    assert choice(256, 64, 58, 128, 3, 2) == 3
    assert choice(256, 64, 56, 128, 1, 2) == 3
    assert choice(256, 512, 9, 512, 3, 1) == 3
    assert choice(256, 3, 230, 64, 7, 2) in (1, 2)
    assert choice(32, 3, 36, 32, 5, 1) in (1, 2)


@pytest.mark.parametrize("kernel", [1, 2, 3])
def test_split_expand_keeps_the_other_operand(ops, kernel):
    """rexsc_sc_conv2d_expand with one null operand leaves the other operand's streams in the workspace: weights
    expanded once serve several activation tensors (C ABI called the way bench.py does)."""
    import ctypes as C
    from rexsc_b200 import _lib
    lib = _lib.load()
    N, Cin, H, Cout, K = 3, 64, 10, 40, 3
    g = torch.Generator().manual_seed(5)
    xs = [torch.rand(N, Cin, H, H, generator=g).cuda().contiguous(memory_format=torch.channels_last) for _ in range(2)]
    w = (torch.randn(Cout, Cin, K, K, generator=g) * 0.1).clamp(-1, 1).cuda().contiguous(memory_format=torch.channels_last)
    d = _lib.ScConvDesc()
    d.batch, d.c_in, d.h_in, d.w_in, d.c_out, d.kh, d.kw = N, Cin, H, H, Cout, K, K
    d.stride_h = d.stride_w = 1
    d.act_channels_last = d.w_channels_last = d.out_channels_last = 1
    d.bit_length, d.lfsr_length, d.bin_config, d.gen_config, d.xnor = 32, -1, 1, 1, 1
    d.prog_total_width, d.prog_load_width, d.prog_load_wait = PROG
    d.kernel = kernel
    nbytes = lib.rexsc_sc_conv2d_workspace_size(C.byref(d))
    ws = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    vp = lambda t: C.c_void_p(t.data_ptr())
    oh = H - K + 1

    def outputs():
        pos = torch.empty((N, Cout, oh, oh), dtype=torch.int16, device="cuda", memory_format=torch.channels_last)
        return pos, torch.empty_like(pos)

    assert lib.rexsc_sc_conv2d_expand(C.byref(d), None, None, vp(ws), nbytes, st) == -1        # REXSC_E_BAD_ARG
    assert lib.rexsc_sc_conv2d_expand(C.byref(d), None, vp(w), vp(ws), nbytes, st) == 0        # weights once
    for x in xs:
        assert lib.rexsc_sc_conv2d_expand(C.byref(d), vp(x), None, vp(ws), nbytes, st) == 0    # activations per call
        pos, neg = outputs()
        assert lib.rexsc_sc_conv2d_accumulate(C.byref(d), vp(pos), vp(neg), vp(ws), nbytes, st) == 0
        ws2 = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
        rpos, rneg = outputs()
        assert lib.rexsc_sc_conv2d_fwd(C.byref(d), vp(x), vp(w), vp(rpos), vp(rneg), vp(ws2), nbytes, st) == 0
        torch.cuda.synchronize()
        assert torch.equal(pos, rpos) and torch.equal(neg, rneg)


def test_randomised_tensor_kernel_vs_direct(ops):
    """40 seeded random layer shapes in the tensor-core kernel's range (32..256 input channels, 1x1 / 2x2 / 3x3
    filters, stride 1 or 2, ragged output channels, up to 40 images): persistent tile loops with partial last tiles,
    slot-split tiles, residue planes and odd channel-word counts all occur.  The direct kernel is the reference."""
    import random

    rng = random.Random(7)
    ran = 0
    for trial in range(40):
        K = rng.choice([1, 3, 3, 3, 2])
        stride = rng.choice([1, 1, 2])
        pad = rng.choice([0, 1]) if K > 1 else 0
        Cin = rng.choice([32, 48, 64, 96, 128, 160, 256])
        Cout = rng.choice([8, 64, 64, 128, 192, 70])
        H, W, N = rng.randint(max(K, 4), 40), rng.randint(max(K, 4), 40), rng.randint(1, 40)
        L = rng.choice([32, 32, 64])
        or_n = rng.choice([1, 2, 2, 3, 51201])
        cl = rng.random() < 0.7
        g = torch.Generator(device="cuda").manual_seed(trial)
        x = torch.rand(N, Cin, H, W, device="cuda", generator=g)
        w = (torch.randn(Cout, Cin, K, K, device="cuda", generator=g) * 0.05).clamp(-1, 1)
        if cl:
            x = x.contiguous(memory_format=torch.channels_last)
            w = w.contiguous(memory_format=torch.channels_last)
        got = _run_or_skip_unsupported(lambda: run_ours(ops, x, w, L, pad, stride, or_n, True, "tensor"), "tensor")
        if got is None:
            continue
        ref = run_ours(ops, x, w, L, pad, stride, or_n, True, "direct")
        what = f"trial {trial}: {(N, Cin, H, W, Cout, K, pad, stride, L, or_n, cl)}"
        assert torch.equal(got[0], ref[0]) and torch.equal(got[1], ref[1]), what
        ran += 1
    assert ran >= 30


@pytest.mark.parametrize("kernel", ["auto", "tiled", "direct"])
def test_prepared_conv_reuses_weight_streams(ops, kernel):
    """ops.PreparedConv expands the weights once; every call equals the one-shot op on the same tensors."""
    g = torch.Generator().manual_seed(9)
    w = (torch.randn(64, 64, 3, 3, generator=g) * 0.1).clamp(-1, 1).cuda().contiguous(memory_format=torch.channels_last)
    xs = [torch.rand(5, 64, 12, 12, generator=g).cuda().contiguous(memory_format=torch.channels_last) for _ in range(3)]
    args = (32, -1, (1, 1), (2, 2), PROG, 1, 1, True)
    ops.set_conv_kernel(kernel)
    try:
        conv = ops.PreparedConv(w, xs[0].shape, xs[0].dtype, True, *args)
        for x in xs:
            pos, neg = conv(x)
            rpos, rneg = ops.conv2d_generic_general_split_acc(x, w, 32, -1, 16, (1, 1), (2, 2), PROG, 1, 1, True, False)
            assert torch.equal(pos, rpos) and torch.equal(neg, rneg)
        with pytest.raises(ValueError):
            conv(xs[0][:, :, :11])   # another shape needs another object
    finally:
        ops.set_conv_kernel("auto")


def test_device_timeout_status_is_decoded(ops):
    """A non-zero status word at the head of a workspace (what a bounded device-side wait leaves when it gives up)
    is reported as REXSC_E_DEVICE_TIMEOUT.  The word is written from the host; no kernel runs."""
    import ctypes as C

    from rexsc_b200 import _lib

    lib = _lib.load()
    ws = torch.zeros(1024, dtype=torch.uint8, device="cuda")
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.rexsc_workspace_status(C.c_void_p(ws.data_ptr()), st) == 0
    ws[:4] = torch.tensor([4, 0, 0, 0], dtype=torch.uint8, device="cuda")
    assert lib.rexsc_workspace_status(C.c_void_p(ws.data_ptr()), st) == -6
    with pytest.raises(RuntimeError, match="REXSC_E_DEVICE_TIMEOUT"):
        _lib.check(-6, "status")
    assert lib.rexsc_workspace_status(None, st) == -1
