"""TEST INFRASTRUCTURE: modules named like the reference's extensions, backed by the CPU oracle.

Lets the CPU-only tests run the reference's unchanged front end (and the training harness around it, with gloo
ranks) in a container without a GPU.  The product never imports this file; on a GPU the same names resolve to
``rexsc_b200/dropin``.
"""
import sys
import types

import torch

import oracle


def _conv_split(input, weight, *args):
    p, n = oracle.conv2d_generic_general_split(input, weight, *args)
    return [p, n]


def _conv(input, weight, *args):
    p, n = oracle.conv2d_generic_general_split(input, weight, *args)
    return p - n


def _like(t_double, like, dtype):
    return t_double.to(dtype).reshape(like.shape)


def _orn_fwd(x, or_n):
    return _like(oracle.orn_forward(x, or_n), x, torch.float32)


def _orn_bwd(g, x, or_n):
    return _like(oracle.orn_backward(g, x.half(), or_n), g, torch.float32)


def _both_fwd(p, n, bias, std, or_n):
    mp, sp = oracle.bias_std_moments(p, or_n, bias.cpu().numpy(), std.cpu().numpy())
    mn, sn = oracle.bias_std_moments(n, or_n, bias.cpu().numpy(), std.cpu().numpy())
    out = mp - mn + torch.sqrt(sp * sp + sn * sn) * torch.randn(mp.shape, dtype=torch.float64)
    return _like(out, p, torch.float32)


def _both_bwd(g, p, n, bias, or_n):
    gp = oracle.bias_std_backward(g, p.half(), or_n, bias.cpu().numpy())
    gn = oracle.bias_std_backward(-g, n.half(), or_n, bias.cpu().numpy())
    return [_like(gp, g, torch.float32), _like(gn, g, torch.float32)]


def _single_fwd(x, bias, std, or_n):
    m, s = oracle.bias_std_moments(x.half(), or_n, bias.cpu().numpy(), std.cpu().numpy())
    return _like(m + s * torch.randn(m.shape, dtype=torch.float64), x, torch.float16)


def _single_bwd(g, x, bias, or_n):
    return _like(oracle.bias_std_backward(g, x.half(), or_n, bias.cpu().numpy()), g, torch.float32)


def install():
    """Put oracle-backed ``sc_extension_cuda`` / ``fixed_extension_cuda`` (+ the two CPU names) into sys.modules."""
    sc = types.ModuleType("sc_extension_cuda")
    sc.conv2d_generic_general_split_acc = _conv_split
    sc.conv2d_generic_general_acc = _conv
    sc.linear_generic_general_acc = lambda *a: list(oracle.linear_generic_general(*a))
    sc.or_approx_n_forward_acc = _orn_fwd
    sc.or_approx_n_backward_acc = _orn_bwd
    sc.or_approx_n_forward_bias_std_both_acc = _both_fwd
    sc.or_approx_n_backward_bias_std_both_acc = _both_bwd
    sc.or_approx_n_forward_bias_std_acc = _single_fwd
    sc.or_approx_n_backward_bias_std_acc = _single_bwd
    fx = types.ModuleType("fixed_extension_cuda")
    fx.conv2d_saturate_acc = lambda *a: oracle.conv2d_saturate(*a)
    sys.modules["sc_extension_cuda"] = sc
    sys.modules["fixed_extension_cuda"] = fx
    sys.modules["sc_extension"] = types.ModuleType("sc_extension")
    sys.modules["fixed_extension"] = types.ModuleType("fixed_extension")
    return sc, fx
