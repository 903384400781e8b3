"""GPU parity of the FXP saturating conv (through the C-ABI): bit-exact against the golden vectors produced by
the reference's CPU extension and against the oracle's restatement of the GPU kernel (K padded to 8)."""
import numpy as np
import pytest
import torch

from helpers import conv_inputs, from128, golden_cases, load_golden

pytestmark = pytest.mark.gpu


def test_golden_reference_cpu_vectors(ops):
    g = load_golden("fxp_conv_ref_cpu.npz")
    for name in golden_cases(g):
        N, Cin, H, W, Cout, K, pad, stride, add, p_in, p_out = (int(v) for v in g[name + "/args"])
        x, w = from128(g[name + "/x128"]), from128(g[name + "/w128"])
        y = ops.conv2d_saturate_acc(x.cuda(), w.cuda(), add, p_in, p_out, (pad, pad), (stride, stride))
        assert y.dtype == torch.int32 and y.is_contiguous()
        assert np.array_equal(y.cpu().numpy(), g[name + "/y"]), name


CASES = [
    # N, Cin, H, W, Cout, K, pad, stride, add_config, p_in, p_out, wscale
    (4, 3, 32, 32, 32, 5, 2, 1, 0, 5, 24, 0.1),      # TinyConv layer 1 (closed form)
    (4, 32, 16, 16, 32, 5, 2, 1, 0, 5, 24, 0.1),     # layer 2
    (4, 32, 8, 8, 64, 5, 2, 1, 0, 5, 24, 0.1),       # layer 3
    (8, 64, 4, 4, 10, 4, 0, 1, 0, 7, 24, 0.1),       # last layer, 7-bit
    (2, 5, 9, 11, 7, 3, 1, 2, 0, 6, 24, 0.3),        # ragged everything, K = 45 (padded to 48)
    (1, 16, 6, 6, 8, 3, 1, 1, 0, 7, 16, 0.15),       # cap 2^16 reached (closed form with saturation)
    (1, 13, 6, 6, 8, 3, 1, 1, 0, 7, 10, 0.05),       # precision_diff = 4, K = 117 not a multiple of 8
    (1, 13, 6, 6, 8, 3, 1, 1, 1, 5, 24, 0.1),        # simulated OR add
    (1, 13, 6, 6, 8, 3, 1, 1, 2, 5, 24, 0.1),        # simulated OR-2 pairs, odd K
    (2, 8, 7, 7, 6, 3, 0, 1, 0, 3, 24, 0.5),         # tiny precision
]


@pytest.mark.parametrize("kernel", ["cuda", "tensor", "tensor_unswizzled"])
@pytest.mark.parametrize("case", CASES)
def test_parity_vs_oracle(ops, oracle, case, kernel):
    N, Cin, H, W, Cout, K, pad, stride, add, p_in, p_out, ws = case
    closed_form = add == 0 and 2 * p_in <= p_out
    if kernel.startswith("tensor") and not closed_form:
        pytest.skip("the tensor-core kernel only implements the closed form")
    x, w = conv_inputs(N, Cin, H, W, Cout, K, prec=7, seed=int(ws * 100) + Cin, wscale=ws)
    ref = oracle.conv2d_saturate(x, w, add, p_in, p_out, (pad, pad), (stride, stride), pad8=True)
    ops.set_fxp_kernel(kernel)
    try:
        y = ops.conv2d_saturate_acc(x.cuda(), w.cuda(), add, p_in, p_out, (pad, pad), (stride, stride))
    finally:
        ops.set_fxp_kernel("auto")
    assert torch.equal(y.cpu(), ref), f"{case}: {(y.cpu() != ref).sum().item()} of {ref.numel()} differ"


def test_tensor_core_kernel_wide_layers(ops, oracle):
    """More output channels than one CTA chunk (128) and a dot product spanning many 128-byte slabs."""
    for (N, Cin, H, Cout, K) in [(2, 24, 6, 200, 3), (1, 96, 5, 136, 3)]:
        x, w = conv_inputs(N, Cin, H, H, Cout, K, prec=7, seed=Cout, wscale=0.2)
        ref = oracle.conv2d_saturate(x, w, 0, 6, 24, (1, 1), (1, 1))
        ops.set_fxp_kernel("tensor")
        try:
            y = ops.conv2d_saturate_acc(x.cuda(), w.cuda(), 0, 6, 24, (1, 1), (1, 1))
        finally:
            ops.set_fxp_kernel("auto")
        assert torch.equal(y.cpu(), ref)


def test_half_inputs_and_rounding_ties(ops, oracle):
    """round-half-even at exact ties (x*2^p = k + 0.5) and fp16 inputs."""
    x = (torch.arange(0, 2 * 6 * 6 * 4, dtype=torch.float32).reshape(2, 4, 6, 6) % 64 + 0.5) / 64
    w = ((torch.arange(0, 5 * 4 * 9, dtype=torch.float32).reshape(5, 4, 3, 3) % 33 - 16) + 0.5) / 32
    ref = oracle.conv2d_saturate(x, w, 0, 5, 24, (1, 1), (1, 1))
    for dt in (torch.float32, torch.float16):
        y = ops.conv2d_saturate_acc(x.cuda().to(dt), w.cuda().to(dt), 0, 5, 24, (1, 1), (1, 1))
        assert torch.equal(y.cpu(), ref), dt


def test_channels_last_input_is_read_logically(ops, oracle):
    x, w = conv_inputs(2, 8, 8, 8, 6, 3, seed=12)
    ref = oracle.conv2d_saturate(x, w, 0, 5, 24, (1, 1), (1, 1))
    y = ops.conv2d_saturate_acc(x.cuda().contiguous(memory_format=torch.channels_last), w.cuda(), 0, 5, 24, (1, 1),
                                (1, 1))
    assert torch.equal(y.cpu(), ref)


def test_full_size_properties(ops):
    """TinyConv layer 2 at the benchmark batch (256): determinism, sign symmetry and additivity over input
    channels below the cap (the closed form is a plain sum there)."""
    g = torch.Generator().manual_seed(1)
    x = torch.rand(256, 32, 16, 16, generator=g).cuda()
    w = (torch.randn(32, 32, 5, 5, generator=g) * 0.1).clamp(-1, 1).cuda()
    args = (0, 5, 24, (2, 2), (1, 1))
    y1 = ops.conv2d_saturate_acc(x, w, *args)
    y2 = ops.conv2d_saturate_acc(x, w, *args)
    assert torch.equal(y1, y2)
    assert torch.equal(ops.conv2d_saturate_acc(x, -w, *args), -y1)
    ya = ops.conv2d_saturate_acc(x[:, :16].contiguous(), w[:, :16].contiguous(), *args)
    yb = ops.conv2d_saturate_acc(x[:, 16:].contiguous(), w[:, 16:].contiguous(), *args)
    assert torch.equal(ya + yb, y1)
