"""Parity against the reference's OWN GPU extensions, compiled unchanged for sm_100 by
``python oracle/build_ref.py --gpu`` (skipped when oracle/_ref does not hold them).  This is the only check that
executes the reference's XNOR generator and its point-wise CUDA kernels; shapes stay inside what the reference's
front end feeds them."""
import os
import sys

import pytest
import torch

from helpers import conv_inputs

pytestmark = pytest.mark.gpu

PROG = (7, 8, 1)


@pytest.fixture(scope="module")
def ref_gpu():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import build_ref

    try:
        mods = build_ref.load_gpu()
    except Exception as exc:  # built for another torch / CUDA runtime
        pytest.skip(f"reference GPU extension does not load here: {exc}")
    if mods is None:
        pytest.skip("oracle/_ref holds no reference GPU extension (python oracle/build_ref.py --gpu)")
    return mods


CONV_CASES = [
    # N, Cin, H, W, Cout, K, pad, stride, L, or_n, channels_last
    (4, 3, 32, 32, 32, 5, 2, 1, 32, 1, False),      # config-1 shape at a small batch
    (4, 64, 14, 14, 64, 3, 1, 1, 32, 2, True),
    (2, 64, 14, 14, 128, 3, 1, 2, 32, 2, True),
    (2, 64, 14, 14, 128, 1, 0, 2, 32, 2, True),
    (2, 64, 10, 10, 64, 3, 1, 1, 64, 3, True),
    (2, 70, 9, 9, 40, 3, 1, 1, 32, 2, False),
    (2, 64, 4, 4, 10, 4, 0, 1, 128, 1, False),
    (2, 40, 7, 7, 9, 3, 1, 1, 4, 2, False),         # 4-bit streams: 3-bit LFSR, values scaled by 4
]


@pytest.mark.parametrize("xnor", [True, False])
@pytest.mark.parametrize("case", CONV_CASES)
def test_sc_conv_matches_reference_gpu_kernels(ops, ref_gpu, case, xnor):
    N, Cin, H, W, Cout, K, pad, stride, L, or_n, cl = case
    x, w = conv_inputs(N, Cin, H, W, Cout, K, prec=7, seed=sum(case))
    x = torch.nn.functional.pad(x, (pad, pad, pad, pad)).cuda()
    w = w.cuda()
    if cl:
        x = x.contiguous(memory_format=torch.channels_last)
        w = w.contiguous(memory_format=torch.channels_last)
    args = (L, -1, 16, (0, 0), (stride, stride), PROG, or_n - 1, 1, xnor, False)
    rp, rn = ref_gpu[0].conv2d_generic_general_split_acc(x, w, *args)
    torch.cuda.synchronize()
    p, n = ops.conv2d_generic_general_split_acc(x, w, *args)
    assert p.stride() == rp.stride()
    assert torch.equal(p, rp) and torch.equal(n, rn), f"{case} xnor={xnor}"


# The layer shapes of the two ImageNet configurations at their full batch: (N, Cin, H, Cout, K, stride, pad, L, or_n).
# ResNet-18, batch 256, 32-bit streams, OR-2: the six distinct SC conv shapes; ResNet-34, batch 192, 64-bit, OR-3.
FULL_SIZE_CASES = [
    (256, 64, 56, 64, 3, 1, 1, 32, 2), (256, 64, 56, 128, 3, 2, 1, 32, 2), (256, 128, 28, 128, 3, 1, 1, 32, 2),
    (256, 256, 14, 256, 3, 1, 1, 32, 2), (256, 512, 7, 512, 3, 1, 1, 32, 2), (256, 64, 56, 128, 1, 2, 0, 32, 2),
    (256, 128, 28, 256, 3, 2, 1, 32, 2), (256, 256, 14, 512, 3, 2, 1, 32, 2), (256, 256, 14, 512, 1, 2, 0, 32, 2),
    (192, 64, 56, 64, 3, 1, 1, 64, 3), (192, 128, 28, 256, 3, 2, 1, 64, 3), (192, 512, 7, 512, 3, 1, 1, 64, 3),
]


@pytest.mark.parametrize("case", FULL_SIZE_CASES)
def test_sc_conv_full_size_matches_reference_gpu_kernels(ops, ref_gpu, case):
    """Channels_last, XNOR generator (the front end's setting), full batch: every output count of the persistent
    tensor-core path (many tiles per CTA, compact grid chosen by the border check on caller-padded inputs, atomically
    added cut tiles) against the reference's kernels, bit for bit."""
    N, C, H, Co, K, s, p, L, or_n = case
    g = torch.Generator(device="cuda").manual_seed(sum(case))
    x = torch.rand(N, C, H + 2 * p, H + 2 * p, device="cuda", generator=g)
    x = ((x * 128).round() / 128).contiguous(memory_format=torch.channels_last)
    if p:
        x[:, :, :p], x[:, :, -p:], x[:, :, :, :p], x[:, :, :, -p:] = 0, 0, 0, 0    # the zero border F.pad leaves
    w = (torch.randn(Co, C, K, K, device="cuda", generator=g) * 0.1).clamp(-1, 1)
    w = ((w * 128).round() / 128).contiguous(memory_format=torch.channels_last)
    args = (L, -1, 16, (0, 0), (s, s), PROG, or_n - 1, 1, True, False)
    rp, rn = ref_gpu[0].conv2d_generic_general_split_acc(x, w, *args)
    torch.cuda.synchronize()
    pos, neg = ops.conv2d_generic_general_split_acc(x, w, *args)
    assert ops.workspace_status() == 0
    assert pos.stride() == rp.stride()
    assert torch.equal(pos, rp) and torch.equal(neg, rn), case
    del rp, rn, pos, neg, x, w
    torch.cuda.empty_cache()


# The reference's GPU *linear* op is not executed here: its translation unit keeps its own copy of the scratch
# pointers but shares the "already allocated" flag with the conv unit (sc_device.cuh:711-714, sc_device.cu:3,
# sc_cuda_matmul.cu:634-644), so calling it after a conv in the same process dereferences unallocated buffers.
# SC linear parity is pinned by the reference CPU extension's vectors instead (tests/test_gpu_sc_conv.py), which
# the reference's GPU generator equals by construction (both ignore xnor and seed by channel).


@pytest.mark.parametrize("or_n", [1, 2, 3, 4])
def test_pointwise_matches_reference_gpu_kernels(ops, ref_gpu, or_n):
    """Same fp32 operation order and the same hardware exp: bit-identical outputs where no noise is drawn."""
    g = torch.Generator().manual_seed(or_n)
    s = (torch.rand(3, 16, 9, 9, generator=g) * 5).cuda()
    grad = torch.randn(3, 16, 9, 9, generator=g).cuda()
    sc = ref_gpu[0]
    assert torch.equal(ops.or_approx_n_forward_acc(s, or_n), sc.or_approx_n_forward_acc(s, or_n))
    assert torch.equal(ops.or_approx_n_forward_acc(s.half(), or_n), sc.or_approx_n_forward_acc(s.half(), or_n))
    assert torch.equal(ops.or_approx_n_backward_acc(grad, s, or_n), sc.or_approx_n_backward_acc(grad, s, or_n))
    bias = torch.tensor([0.01, -0.05, 0.02, 0.003, -0.001, 0.0002, 0, 0, 0, 0, 0]).cuda()
    zero = torch.zeros(11).cuda()
    p, n = s, s.flip(0).contiguous()
    ours = ops.or_approx_n_forward_bias_std_both_acc(p, n, bias, zero, or_n)
    ref = sc.or_approx_n_forward_bias_std_both_acc(p, n, bias, zero, or_n)
    assert torch.equal(ours, ref)
    gp, gn = ops.or_approx_n_backward_bias_std_both_acc(grad, p, n, bias, or_n)
    rgp, rgn = sc.or_approx_n_backward_bias_std_both_acc(grad, p, n, bias, or_n)
    assert torch.equal(gp, rgp) and torch.equal(gn, rgn)
    assert torch.equal(ops.or_approx_n_backward_bias_std_acc(grad, s, bias, or_n),
                       sc.or_approx_n_backward_bias_std_acc(grad, s, bias, or_n))
    assert torch.equal(ops.or_approx_n_forward_bias_std_acc(s, bias, zero, or_n),
                       sc.or_approx_n_forward_bias_std_acc(s, bias, zero, or_n))


def test_injection_statistics_match_reference_gpu_kernels(ops, ref_gpu):
    """With noise on only the statistics can agree: same mean and variance as the reference's cuRAND stream."""
    n_elem = 1 << 20
    p = torch.full((n_elem,), 1.3).cuda()
    n = torch.full((n_elem,), 0.4).cuda()
    bias = torch.tensor([0.01, -0.05, 0.02, 0.003, -0.001, 0.0002, 0, 0, 0, 0, 0]).cuda()
    std = torch.tensor([0.02, 0.05, -0.01, 0.002, 0.0, 0.0001, 0, 0, 0, 0, 0]).cuda()
    ours = ops.or_approx_n_forward_bias_std_both_acc(p, n, bias, std, 2).double()
    ref = ref_gpu[0].or_approx_n_forward_bias_std_both_acc(p, n, bias, std, 2).double()
    se = (ref.var().item() / n_elem) ** 0.5
    assert abs(ours.mean().item() - ref.mean().item()) < 8 * se
    assert abs(ours.var().item() / ref.var().item() - 1) < 0.02


FXP_CASES = [(4, 3, 32, 32, 32, 5, 2, 1, 0, 5, 24), (4, 32, 16, 16, 32, 5, 2, 1, 0, 5, 24),
             (4, 64, 4, 4, 10, 4, 0, 1, 0, 7, 24), (1, 13, 6, 6, 8, 3, 1, 1, 0, 7, 10), (1, 13, 6, 6, 8, 3, 1, 1, 1, 5, 24)]


@pytest.mark.parametrize("case", FXP_CASES)
def test_fxp_matches_reference_gpu_kernel(ops, ref_gpu, case):
    N, Cin, H, W, Cout, K, pad, stride, add, p_in, p_out = case
    x, w = conv_inputs(N, Cin, H, W, Cout, K, prec=7, seed=sum(case))
    x, w = x.cuda(), w.cuda()
    ref = ref_gpu[1].conv2d_saturate_acc(x, w, add, p_in, p_out, (pad, pad), (stride, stride))
    torch.cuda.synchronize()
    ours = ops.conv2d_saturate_acc(x, w, add, p_in, p_out, (pad, pad), (stride, stride))
    assert torch.equal(ours, ref), case
