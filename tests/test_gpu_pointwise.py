"""GPU tests of the point-wise kernels through the C-ABI: OR-n activation forward/backward, the fused
bias/std (calibration + error injection) ops and their single-sided variants.

Tolerances: the kernels evaluate fp32 with the hardware exp approximation, the oracle is double precision;
forward values agree to 2e-6 absolute + 1e-5 relative (outputs are O(1)), gradients to 1e-3 relative as the
parity contract states.  With all coefficients zero the fused op must equal f_n(pos) - f_n(neg) exactly, and
noise statistics are checked in mean and variance."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

OR_NS = [1, 2, 3, 4]


def sums(n_elem, seed, dtype=torch.float32, hi=6.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.rand(n_elem, generator=g) * hi).to(dtype)


@pytest.mark.parametrize("or_n", OR_NS)
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_orn_forward(ops, oracle, or_n, dtype):
    for n_elem in (1, 3, 4, 1000, 4099, 1 << 18):
        s = sums(n_elem, or_n, dtype)
        out = ops.or_approx_n_forward_acc(s.cuda(), or_n)
        assert out.dtype == torch.float32 and out.shape == s.shape
        ref = oracle.orn_forward(s.double(), or_n)
        assert torch.allclose(out.cpu().double(), ref, rtol=1e-5, atol=2e-6), (or_n, dtype, n_elem)


@pytest.mark.parametrize("or_n", OR_NS)
def test_orn_forward_layouts_and_views(ops, oracle, or_n):
    g = torch.Generator().manual_seed(5)
    x = (torch.rand(3, 8, 5, 7, generator=g) * 4).cuda()
    ref = oracle.orn_forward(x.cpu().double(), or_n).float()
    for t in (x, x.contiguous(memory_format=torch.channels_last), x[:, ::2], x.permute(0, 2, 3, 1)):
        out = ops.or_approx_n_forward_acc(t, or_n)
        r = oracle.orn_forward(t.cpu().double(), or_n).float()
        assert out.shape == t.shape
        assert torch.allclose(out.cpu(), r, rtol=1e-5, atol=2e-6)
    # misaligned base pointer takes the scalar path
    flat = (torch.rand(1027, generator=g) * 4).cuda()
    out = ops.or_approx_n_forward_acc(flat[1:], or_n)
    assert torch.allclose(out.cpu(), oracle.orn_forward(flat[1:].cpu().double(), or_n).float(), rtol=1e-5, atol=2e-6)
    assert ref is not None


@pytest.mark.parametrize("or_n", OR_NS)
def test_orn_backward(ops, oracle, or_n):
    s = sums(5003, 10 + or_n)
    g = torch.randn(5003, generator=torch.Generator().manual_seed(1))
    out = ops.or_approx_n_backward_acc(g.cuda(), s.cuda(), or_n)
    assert out.dtype == torch.float32
    # the reference rounds the saved sum to fp16 before differentiating (sc_cuda_pw.cu:775)
    ref = oracle.orn_backward(g.double(), s.half().double(), or_n)
    assert torch.allclose(out.cpu().double(), ref, rtol=1e-3, atol=1e-6)
    # and it stays within the contract's 1e-3 of the unrounded derivative scale
    ref_exact = oracle.orn_backward(g.double(), s.double(), or_n)
    assert (out.cpu().double() - ref_exact).abs().max() <= 3e-3 * g.abs().max()
    with pytest.raises(RuntimeError):
        ops.or_approx_n_backward_acc(g.cuda().half(), s.cuda(), or_n)


@pytest.mark.parametrize("or_n", OR_NS)
def test_fused_both_forward_exact_without_injection(ops, or_n):
    """Zero bias and std coefficients: exactly f_n(pos) - f_n(neg), bit for bit with the plain kernel."""
    p, n = sums(70001, 20 + or_n).cuda(), sums(70001, 30 + or_n).cuda()
    zero = torch.zeros(11).cuda()
    out = ops.or_approx_n_forward_bias_std_both_acc(p, n, zero, zero, or_n)
    plain = ops.or_approx_n_forward_acc(p, or_n) - ops.or_approx_n_forward_acc(n, or_n)
    assert torch.equal(out, plain)


@pytest.mark.parametrize("or_n", [1, 2, 3])
def test_fused_both_forward_bias_and_noise_statistics(ops, oracle, or_n):
    ops.manual_seed(1234)
    bias = torch.tensor([0.01, -0.05, 0.02, 0.003, -0.001, 0.0002, 0, 0, 0, 0, 0])
    std = torch.tensor([0.02, 0.05, -0.01, 0.002, 0.0, 0.0001, 0, 0, 0, 0, 0])
    n_elem = 1 << 20
    # constant inputs: every element draws from the same Gaussian
    sp, sn = 1.7, 0.6
    p = torch.full((n_elem,), sp).cuda()
    n = torch.full((n_elem,), sn).cuda()
    out = ops.or_approx_n_forward_bias_std_both_acc(p, n, bias.cuda(), std.cuda(), or_n).cpu().double()
    mp, sdp = oracle.bias_std_moments(torch.tensor([sp]), or_n, bias.numpy(), std.numpy())
    mn, sdn = oracle.bias_std_moments(torch.tensor([sn]), or_n, bias.numpy(), std.numpy())
    mean_ref = float(mp - mn)
    var_ref = float(sdp ** 2 + sdn ** 2)
    se = (var_ref / n_elem) ** 0.5
    assert abs(out.mean().item() - mean_ref) < 6 * se + 1e-6
    assert abs(out.var().item() / var_ref - 1) < 0.01
    z = (out - mean_ref) / var_ref ** 0.5
    assert abs((z ** 3).mean().item()) < 0.02 and abs((z ** 4).mean().item() - 3) < 0.05   # Gaussian shape
    # successive calls draw fresh noise; re-seeding reproduces the first call
    out2 = ops.or_approx_n_forward_bias_std_both_acc(p, n, bias.cuda(), std.cuda(), or_n).cpu().double()
    assert not torch.equal(out, out2)
    assert abs(torch.corrcoef(torch.stack([out, out2]))[0, 1].item()) < 0.01
    ops.manual_seed(1234)
    out3 = ops.or_approx_n_forward_bias_std_both_acc(p, n, bias.cuda(), std.cuda(), or_n).cpu().double()
    assert torch.equal(out, out3)
    # std = 0: deterministic and equal to the mean model
    zero = torch.zeros(11)
    det = ops.or_approx_n_forward_bias_std_both_acc(p[:4096], n[:4096], bias.cuda(), zero.cuda(), or_n).cpu().double()
    assert torch.allclose(det, torch.full_like(det, mean_ref), rtol=1e-5, atol=2e-6)


@pytest.mark.parametrize("or_n", OR_NS)
def test_fused_both_backward(ops, oracle, or_n):
    bias = np.array([0.01, -0.05, 0.02, 0.003, -0.001, 0.0002])
    p, n = sums(4097, 40 + or_n), sums(4097, 50 + or_n)
    g = torch.randn(4097, generator=torch.Generator().manual_seed(2))
    b = torch.tensor(bias, dtype=torch.float32).cuda()
    gp, gn = ops.or_approx_n_backward_bias_std_both_acc(g.cuda(), p.cuda(), n.cuda(), b, or_n)
    rp = oracle.bias_std_backward(g.double(), p.half().double(), or_n, bias)
    rn = oracle.bias_std_backward(-g.double(), n.half().double(), or_n, bias)
    assert torch.allclose(gp.cpu().double(), rp, rtol=1e-3, atol=1e-6)
    assert torch.allclose(gn.cpu().double(), rn, rtol=1e-3, atol=1e-6)
    # fp16 saved sums (autocast) give the same numbers
    gp16, gn16 = ops.or_approx_n_backward_bias_std_both_acc(g.cuda(), p.cuda().half(), n.cuda().half(), b, or_n)
    assert torch.equal(gp16, gp) and torch.equal(gn16, gn)


@pytest.mark.parametrize("or_n", OR_NS)
def test_single_sided_variants(ops, oracle, or_n):
    bias = np.array([0.02, -0.03, 0.01, 0.002, 0.0, 0.0001])
    s = sums(8191, 60 + or_n)
    zero = torch.zeros(6).cuda()
    b = torch.tensor(bias, dtype=torch.float32).cuda()
    out = ops.or_approx_n_forward_bias_std_acc(s.cuda(), b, zero, or_n)
    assert out.dtype == torch.float16
    mean, _ = oracle.bias_std_moments(s.half().double(), or_n, bias, np.zeros(6))
    assert torch.allclose(out.cpu().double(), mean, rtol=2e-3, atol=2e-3)   # fp16 output
    g = torch.randn(8191, generator=torch.Generator().manual_seed(3))
    gi = ops.or_approx_n_backward_bias_std_acc(g.cuda(), s.cuda(), b, or_n)
    ref = oracle.bias_std_backward(g.double(), s.half().double(), or_n, bias)
    assert torch.allclose(gi.cpu().double(), ref, rtol=1e-3, atol=1e-6)


def test_autograd_contract(ops):
    """The reference wraps the ops in autograd.Functions (utils_functional.py:468-495,559-575); the same
    wrappers on these ops must pass a finite-difference check of the mean model."""
    class OrN(torch.autograd.Function):
        @staticmethod
        def forward(ctx, s, n):
            ctx.n = n
            ctx.save_for_backward(s)
            return ops.or_approx_n_forward_acc(s, n)

        @staticmethod
        def backward(ctx, g):
            (s,) = ctx.saved_tensors
            return ops.or_approx_n_backward_acc(g, s, ctx.n), None

    s = (torch.rand(64, generator=torch.Generator().manual_seed(4)) * 3).cuda().requires_grad_(True)
    y = OrN.apply(s, 2)
    y.sum().backward()
    h = 1e-2
    num = (ops.or_approx_n_forward_acc(s.detach() + h, 2) - ops.or_approx_n_forward_acc(s.detach() - h, 2)) / (2 * h)
    assert torch.allclose(s.grad, num, rtol=2e-3, atol=2e-4)


def test_rejects_unsupported_n(ops):
    x = torch.rand(16).cuda()
    with pytest.raises(ValueError):
        ops.or_approx_n_forward_acc(x, 5)
    with pytest.raises(ValueError):
        ops.or_approx_n_forward_acc(x, 0)
