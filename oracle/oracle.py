"""ctypes front end of the CPU oracle (rexsc_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, __graft_entry__.smoke() and the
cpu_baseline / reference legs of bench.py -- never by the product package.

The functions take the same arguments as the reference's extension ops
(torch_c/sc-extension/sc_cuda.cpp:73-120, fixed_cuda.cpp:24-34) and return CPU
torch tensors, so a parity test reads ``ours(args) == oracle(args)``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "rexsc_oracle.c")
LIB = os.path.join(HERE, "librexsc_oracle.so")

_lib = None


def build(force: bool = False) -> str:
    if force or not os.path.exists(LIB) or os.path.getmtime(LIB) < os.path.getmtime(SRC):
        cc = "/usr/bin/gcc" if os.path.exists("/usr/bin/gcc") else "gcc"
        # no -march=native: the shared object travels to machines with other CPUs
        subprocess.check_call([cc, "-O2", "-fopenmp", "-fPIC", "-shared", "-std=c11", "-o", LIB, SRC, "-lm"])
    return LIB


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(LIB)
        _lib.rexo_orn_fwd.restype = C.c_double
        _lib.rexo_orn_fwd.argtypes = [C.c_double, C.c_int]
        _lib.rexo_orn_bwd.restype = C.c_double
        _lib.rexo_orn_bwd.argtypes = [C.c_double, C.c_int]
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _i64(v):
    return C.c_int64(int(v))


def lfsr_next(v: int, l: int, xnor: bool) -> int:
    return lib().rexo_lfsr_next(int(v), int(l), int(bool(xnor)))


def lfsr_length_for(bit_length: int) -> int:
    return lib().rexo_lfsr_length_for(int(bit_length))


def stream_bits(value, seed, l, xnor, bit_length, gen_config=1, prog_load=(7, 8, 1), is_weight=False):
    out = np.zeros(bit_length * gen_config, dtype=np.uint8)
    lib().rexo_stream_bits(int(value), int(seed), int(l), int(bool(xnor)), int(bit_length), int(gen_config),
                           int(prog_load[0]), int(prog_load[1]), int(prog_load[2]), int(bool(is_weight)), _p(out))
    return out


def _f32(t: torch.Tensor) -> np.ndarray:
    # logical-order contiguous float32 copy; fp16/bf16 -> fp32 is exact
    return np.ascontiguousarray(t.detach().cpu().to(torch.float32).contiguous().numpy())


def _is_channels_last(t: torch.Tensor) -> bool:
    # layout rule of torch_c/sc-extension/sc_cuda_kernel.cu:585-590
    s = t.stride()
    return s[1] == 1 and s[1] * s[2] * s[3] != 1


def quantize_act(x: torch.Tensor, scale: int, rounding="ceil") -> np.ndarray:
    a = _f32(x)
    q = np.empty(a.shape, dtype=np.int32)
    fn = lib().rexo_quantize_act if rounding == "ceil" else lib().rexo_quantize_act_round
    fn(_p(a), _i64(a.size), int(scale), _p(q))
    return q


def quantize_weight(w: torch.Tensor, scale: int, rounding="ceil"):
    a = _f32(w)
    wp = np.empty(a.shape, dtype=np.int32)
    wn = np.empty(a.shape, dtype=np.int32)
    fn = lib().rexo_quantize_weight if rounding == "ceil" else lib().rexo_quantize_weight_round
    fn(_p(a), _i64(a.size), int(scale), _p(wp), _p(wn))
    return wp, wn


def conv2d_generic_general_split(input, weight, bit_length, lfsr_length, z_units, padding, stride, prog_load,
                                 bin_config, gen_config, xnor, mux):
    """Oracle of sc_extension_cuda.conv2d_generic_general_split_acc (sc_cuda.cpp:87-99)."""
    cl = _is_channels_last(input)
    x = torch.nn.functional.pad(input.detach().cpu().float(), (padding[0], padding[0], padding[1], padding[1]))
    scale = bit_length if lfsr_length <= 0 else (1 << lfsr_length)
    aq = quantize_act(x, scale)
    wp, wn = quantize_weight(weight, scale)
    N, Cc, H, W = aq.shape
    Co, _, KH, KW = wp.shape
    OH, OW = (H - KH) // stride[0] + 1, (W - KW) // stride[1] + 1
    op = np.zeros((N, Co, OH, OW), dtype=np.int16)
    on = np.zeros((N, Co, OH, OW), dtype=np.int16)
    rc = lib().rexo_sc_conv2d(_p(aq), _p(wp), _p(wn), N, Cc, H, W, Co, KH, KW, int(stride[0]), int(stride[1]),
                              int(bit_length), int(lfsr_length), int(prog_load[0]), int(prog_load[1]),
                              int(prog_load[2]), int(bin_config), int(gen_config), int(bool(xnor)), _p(op), _p(on))
    if rc != 0:
        raise ValueError(f"oracle rexo_sc_conv2d rejected the arguments (code {rc})")
    tp, tn = torch.from_numpy(op), torch.from_numpy(on)
    if cl:
        tp = tp.contiguous(memory_format=torch.channels_last)
        tn = tn.contiguous(memory_format=torch.channels_last)
    return tp, tn


def linear_generic_general(input, weight, prog_load, bit_length, lfsr_length, bin_config, gen_config, xnor, mux):
    """Oracle of sc_extension_cuda.linear_generic_general_acc (sc_cuda.cpp:101-120).  The linear
    generators ignore xnor (sc_cuda_matmul.cu:27-57,77-78,177), hence xnor=False below."""
    scale = bit_length if lfsr_length <= 0 else (1 << lfsr_length)
    aq = quantize_act(input, scale)
    wp, wn = quantize_weight(weight, scale)
    B, Cin = aq.shape
    Co = wp.shape[0]
    op = np.zeros((B, Co), dtype=np.int16)
    on = np.zeros((B, Co), dtype=np.int16)
    rc = lib().rexo_sc_conv2d(_p(aq), _p(wp), _p(wn), B, Cin, 1, 1, Co, 1, 1, 1, 1, int(bit_length),
                              int(lfsr_length), int(prog_load[0]), int(prog_load[1]), int(prog_load[2]),
                              int(bin_config), int(gen_config), 0, _p(op), _p(on))
    if rc != 0:
        raise ValueError(f"oracle rexo_sc_conv2d rejected the arguments (code {rc})")
    return torch.from_numpy(op), torch.from_numpy(on)


def conv2d_saturate(input, weight, add_config, precision_in, precision_out, padding, stride, pad8=True):
    """Oracle of fixed_extension_cuda.conv2d_saturate_acc (fixed_cuda.cpp:24-34); pad8=False gives
    the CPU twin fixed.cpp:197-238."""
    x = torch.nn.functional.pad(input.detach().cpu().float(), (padding[0], padding[0], padding[1], padding[1]))
    scale = 1 << precision_in
    aq = quantize_act(x, scale, "round")
    wp, wn = quantize_weight(weight, scale, "round")
    N, Cc, H, W = aq.shape
    Co, _, KH, KW = wp.shape
    OH, OW = (H - KH) // stride[0] + 1, (W - KW) // stride[1] + 1
    out = np.zeros((N, Co, OH, OW), dtype=np.int32)
    rc = lib().rexo_fxp_conv2d(_p(aq), _p(wp), _p(wn), N, Cc, H, W, Co, KH, KW, int(stride[0]), int(stride[1]),
                               int(add_config), int(precision_in), int(precision_out), int(bool(pad8)), _p(out))
    if rc != 0:
        raise ValueError(f"oracle rexo_fxp_conv2d rejected the arguments (code {rc})")
    return torch.from_numpy(out)


def orn_forward(s: torch.Tensor, or_n: int) -> torch.Tensor:
    a = np.ascontiguousarray(s.detach().cpu().double().contiguous().numpy())
    out = np.empty_like(a)
    lib().rexo_orn_fwd_array(_p(a), _i64(a.size), int(or_n), _p(out))
    return torch.from_numpy(out)


def orn_backward(grad: torch.Tensor, s: torch.Tensor, or_n: int) -> torch.Tensor:
    g = np.ascontiguousarray(grad.detach().cpu().double().contiguous().numpy())
    a = np.ascontiguousarray(s.detach().cpu().double().contiguous().numpy())
    out = np.empty_like(a)
    lib().rexo_orn_bwd_array(_p(g), _p(a), _i64(a.size), int(or_n), _p(out))
    return torch.from_numpy(out)


def bias_std_moments(s: torch.Tensor, or_n: int, bias_coef, std_coef):
    """Mean and std of y = x + B(x) + S(x) eps with x = f_n(s)  (sc_device.cuh:507-528)."""
    a = np.ascontiguousarray(s.detach().cpu().double().contiguous().numpy())
    b = np.ascontiguousarray(np.asarray(bias_coef, dtype=np.float64)[:6])
    c = np.ascontiguousarray(np.asarray(std_coef, dtype=np.float64)[:6])
    mean = np.empty_like(a)
    sig = np.empty_like(a)
    lib().rexo_bias_std_moments(_p(a), _i64(a.size), int(or_n), _p(b), _p(c), _p(mean), _p(sig))
    return torch.from_numpy(mean), torch.from_numpy(sig)


def bias_std_backward(grad: torch.Tensor, s: torch.Tensor, or_n: int, bias_coef) -> torch.Tensor:
    g = np.ascontiguousarray(grad.detach().cpu().double().contiguous().numpy())
    a = np.ascontiguousarray(s.detach().cpu().double().contiguous().numpy())
    b = np.ascontiguousarray(np.asarray(bias_coef, dtype=np.float64)[:6])
    out = np.empty_like(a)
    lib().rexo_bias_std_bwd_array(_p(g), _p(a), _i64(a.size), int(or_n), _p(b), _p(out))
    return torch.from_numpy(out)


def counts_to_value(pos: torch.Tensor, neg: torch.Tensor, bit_length: int, dtype=torch.float32):
    """The caller's arithmetic on the int16 counts, step by step as eager PyTorch runs it
    (utils_functional.py:1181-1182 casts, :1273-1274 divisions, :1324 difference)."""
    vp = pos.to(dtype=dtype) / bit_length
    vn = neg.to(dtype=dtype) / bit_length
    return vp, vn, vp - vn


def calib_windows(a_bit: np.ndarray, a_act: np.ndarray, top=None):
    """Window statistics of compute_bias_std_coef (utils_functional.py:901-925) in numpy: for each start of
    ``linspace(0, max(a_bit), 30)`` the elements with ``start <= a_act < start + 0.1`` (scalar rounded to the
    tensor's fp32 as torch's comparison does), ``err = a_bit - a_act`` in fp32, its count, mean and unbiased
    standard deviation (accumulated in float64).  Returns ``(starts, count, mean, std)``; mean / std are NaN
    where the reference skips the window (fewer than two elements).  ``top`` overrides ``max(a_bit)`` (a shard of a
    batch whose maximum was found over all shards)."""
    a_bit = np.asarray(a_bit, dtype=np.float32).reshape(-1)
    a_act = np.asarray(a_act, dtype=np.float32).reshape(-1)
    if top is None:
        top = float(a_bit.max()) if a_bit.size else 0.0
    starts = np.linspace(0, top, 30)
    count = np.zeros(30, dtype=np.int64)
    mean = np.full(30, np.nan)
    std = np.full(30, np.nan)
    err_all = (a_bit - a_act).astype(np.float32)
    for i, start in enumerate(starts):
        sel = (a_act >= np.float32(start)) & (a_act < np.float32(start + 0.1))
        err = err_all[sel].astype(np.float64)
        count[i] = err.size
        if err.size > 1:
            mean[i] = err.mean()
            std[i] = err.std(ddof=1)
    return starts, count, mean, std


def calib_window_sums(a_bit: np.ndarray, a_act: np.ndarray, top=None) -> np.ndarray:
    """``[30, 3]`` float64: element count, sum of err and sum of err^2 per window of calib_windows (the form in which
    shards of a batch can be added up)."""
    a_bit = np.asarray(a_bit, dtype=np.float32).reshape(-1)
    a_act = np.asarray(a_act, dtype=np.float32).reshape(-1)
    if top is None:
        top = float(a_bit.max()) if a_bit.size else 0.0
    out = np.zeros((30, 3))
    err_all = (a_bit - a_act).astype(np.float32).astype(np.float64)
    for i, start in enumerate(np.linspace(0, top, 30)):
        sel = (a_act >= np.float32(start)) & (a_act < np.float32(start + 0.1))
        out[i] = (sel.sum(), err_all[sel].sum(), (err_all[sel] ** 2).sum())
    return out


def compute_bias_std_coef(or_n: int, a_bit: torch.Tensor, a_act: torch.Tensor, order: int = 5):
    """compute_bias_std_coef (utils_functional.py:901-950) on top of calib_windows: polynomial least-squares fits
    of the per-window bias and standard deviation over the window starts; the bias fit is skipped (zeros) when
    ``order >= valid_windows // 5``."""
    if or_n < 0:
        return torch.zeros(order + 1), torch.zeros(order + 1)
    starts, count, mean, std = calib_windows(a_bit.float().numpy(), a_act.float().numpy())
    valid = count > 1
    basis = torch.from_numpy(np.stack([starts[valid] ** i for i in range(order + 1)], axis=1)).float()
    bias_bins = torch.from_numpy(mean[valid]).float()
    std_bins = torch.from_numpy(std[valid]).float()
    if order >= int(valid.sum()) // 5:
        bias_coef = torch.zeros(order + 1)
    else:
        bias_coef = torch.linalg.lstsq(basis, bias_bins)[0]
    std_coef = torch.linalg.lstsq(basis, std_bins)[0]
    return bias_coef, std_coef


def num_threads() -> int:
    return lib().rexo_num_threads()
