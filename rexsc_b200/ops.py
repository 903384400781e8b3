"""Host-side mirror of the reference's extension ops, on top of the C-ABI CUDA library.

Same function names, positional argument lists, dtypes, layouts and return types as the pybind modules
``sc_extension_cuda`` (torch_c/sc-extension/sc_cuda.cpp:122-132) and ``fixed_extension_cuda``
(fixed_cuda.cpp:36-38) of nanocad-lab/rex-sc.  PyTorch is used for device memory and the current stream
only; all arithmetic happens in librexsc_b200.so.  There is no CPU path: tensors must live on a CUDA device.
"""
from __future__ import annotations

import ctypes as C
import os
import threading
from typing import List, Sequence, Tuple

import torch

from . import _lib

_DTYPES = {torch.float32: _lib.F32, torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}
_DEBUG = os.environ.get("REXSC_B200_DEBUG", "0") == "1"
_NVTX = os.environ.get("REXSC_B200_NVTX", "0") == "1"


def _traced(fn):
    """With REXSC_B200_NVTX=1 every op call is an NVTX range named after the op (shows up in Nsight timelines between
    the front end's own torch ranges); otherwise the function is returned untouched."""
    if not _NVTX:
        return fn
    import functools

    @functools.wraps(fn)
    def wrapper(*args, **kwargs):
        torch.cuda.nvtx.range_push("rexsc_b200." + fn.__name__)
        try:
            return fn(*args, **kwargs)
        finally:
            torch.cuda.nvtx.range_pop()
    return wrapper

# conv kernel selection for tests / benchmarks: "auto" | "direct" | "tiled" | "tensor"
_kernel_choice = threading.local()


def set_conv_kernel(name: str) -> None:
    """Force the SC conv kernel ("auto", "direct", "tiled" or "tensor"); results are identical, only speed differs."""
    _kernel_choice.value = {"auto": _lib.KERNEL_AUTO, "direct": _lib.KERNEL_DIRECT, "tiled": _lib.KERNEL_TILED,
                            "tensor": _lib.KERNEL_TENSOR}[name]


def _kernel() -> int:
    return getattr(_kernel_choice, "value", _lib.KERNEL_AUTO)


def set_fxp_kernel(name: str) -> None:
    """Force the FXP conv kernel family: "auto", "cuda" (dp4a / sequential) or "tensor" (tcgen05 int8)."""
    _kernel_choice.fxp = {"auto": 0, "cuda": 1, "tensor": 2, "tensor_unswizzled": 3}[name]


# ---- workspace: one growing byte buffer per (device, stream), owned by torch's caching allocator --------
_workspaces: dict = {}


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def release_workspaces() -> None:
    """Drop the cached scratch buffers (they are re-created on demand)."""
    _workspaces.clear()


def _stream(device) -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _ptr(t: torch.Tensor) -> C.c_void_p:
    return C.c_void_p(t.data_ptr())


def _require_cuda(t: torch.Tensor, what: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{what}: expected a CUDA tensor (rexsc_b200 has no CPU path)")


def _float_kind(t: torch.Tensor) -> torch.Tensor:
    return t if t.dtype in _DTYPES else t.to(torch.float32)


def _is_channels_last(t: torch.Tensor) -> bool:
    # layout rule of torch_c/sc-extension/sc_cuda_kernel.cu:585-590
    s = t.stride()
    return s[1] == 1 and s[1] * s[2] * s[3] != 1


def _dense(t: torch.Tensor, channels_last: bool) -> torch.Tensor:
    return t.contiguous(memory_format=torch.channels_last if channels_last else torch.contiguous_format)


def _flat_dense(t: torch.Tensor) -> torch.Tensor:
    """Tensor whose storage is a dense permutation of its elements (point-wise kernels walk memory order)."""
    if t.is_contiguous() or (t.dim() == 4 and t.is_contiguous(memory_format=torch.channels_last)):
        return t
    if hasattr(t, "is_non_overlapping_and_dense") and t.is_non_overlapping_and_dense():
        return t
    return t.contiguous()


# ---- SC conv2d / linear -------------------------------------------------------------------------------
@_traced
def conv2d_generic_general_split_acc(input: torch.Tensor, weight: torch.Tensor, bit_length: int, lfsr_length: int,
                                     z_units: int, padding: Sequence[int], stride: Sequence[int],
                                     prog_load: Sequence[int], bin_config: int, gen_config: int, xnor: bool,
                                     mux: bool, out=None) -> List[torch.Tensor]:
    """SC conv2d forward, returns [pos, neg] int16 (sc_cuda.cpp:87-99).  ``z_units`` and ``mux`` are accepted
    and unused, as on the reference GPU path (sc_cuda_kernel.cu:565-578).  ``out`` (not in the reference) lets a
    caller supply the two int16 output tensors, in the activation's memory format, instead of fresh ones."""
    _require_cuda(input, "conv2d_generic_general_split_acc")
    _require_cuda(weight, "conv2d_generic_general_split_acc")
    if input.dim() != 4 or weight.dim() != 4 or input.size(1) != weight.size(1):
        raise ValueError("conv2d_generic_general_split_acc: expected input [N,C,H,W] and weight [Co,C,KH,KW]")
    lib = _lib.load()
    dev = input.device
    with torch.cuda.device(dev):
        a_cl = _is_channels_last(input)
        w_cl = _is_channels_last(weight)
        x = _dense(_float_kind(input), a_cl)
        w = _dense(_float_kind(weight), w_cl)
        d = _lib.ScConvDesc()
        d.batch, d.c_in, d.h_in, d.w_in = x.shape
        d.c_out, _, d.kh, d.kw = w.shape
        d.pad_w, d.pad_h = int(padding[0]), int(padding[1])  # padding[0] pads the last dim (sc_cuda.cpp:88)
        d.stride_h, d.stride_w = int(stride[0]), int(stride[1])
        d.act_dtype, d.act_channels_last = _DTYPES[x.dtype], int(a_cl)
        d.w_dtype, d.w_channels_last = _DTYPES[w.dtype], int(w_cl)
        d.out_channels_last = int(a_cl)
        d.bit_length, d.lfsr_length = int(bit_length), int(lfsr_length)
        d.bin_config, d.gen_config, d.xnor = int(bin_config), int(gen_config), int(bool(xnor))
        d.prog_total_width, d.prog_load_width, d.prog_load_wait = (int(v) for v in prog_load)
        d.linear_seeds = 0
        d.kernel = _kernel()
        nbytes = lib.rexsc_sc_conv2d_workspace_size(C.byref(d))
        if nbytes == 0:
            raise ValueError("conv2d_generic_general_split_acc: unsupported shape or configuration")
        oh = (d.h_in + 2 * d.pad_h - d.kh) // d.stride_h + 1
        ow = (d.w_in + 2 * d.pad_w - d.kw) // d.stride_w + 1
        fmt = torch.channels_last if a_cl else torch.contiguous_format
        if out is None:
            pos = torch.empty((d.batch, d.c_out, oh, ow), dtype=torch.int16, device=dev, memory_format=fmt)
            neg = torch.empty((d.batch, d.c_out, oh, ow), dtype=torch.int16, device=dev, memory_format=fmt)
        else:
            pos, neg = out
            for t in (pos, neg):
                if (t.dtype != torch.int16 or t.device != dev or tuple(t.shape) != (d.batch, d.c_out, oh, ow)
                        or not t.is_contiguous(memory_format=fmt)):
                    raise ValueError("conv2d_generic_general_split_acc: `out` tensors must be int16 "
                                     f"[{d.batch},{d.c_out},{oh},{ow}] in the activation's memory format")
        ws = _workspace(dev, nbytes)
        rc = lib.rexsc_sc_conv2d_fwd(C.byref(d), _ptr(x), _ptr(w), _ptr(pos), _ptr(neg), _ptr(ws), ws.numel(),
                                     _stream(dev))
        _lib.check(rc, "rexsc_sc_conv2d_fwd")
        if _DEBUG:
            _lib.check(lib.rexsc_workspace_status(_ptr(ws), _stream(dev)), "rexsc_sc_conv2d_fwd (device status)")
    return [pos, neg]


class PreparedConv:
    """SC conv2d whose weight streams are generated once and reused for every activation tensor of one shape
    (not in the reference, which regenerates both operands' streams on every call -- its results are the same).

    For evaluation / inference loops where the weights do not change between calls::

        conv = ops.PreparedConv(weight, input.shape, input.dtype, channels_last, bit_length, lfsr_length, padding,
                                stride, prog_load, bin_config, gen_config, xnor)
        pos, neg = conv(input)          # as often as needed; build a new object after the weights change

    The object owns its workspace (activation + weight streams of that layer): about the size of the layer's activation
    bit planes -- 220 MB for the largest ResNet-18 layer at batch 256, roughly 1 GB for all 19 layers of that model."""

    def __init__(self, weight: torch.Tensor, input_shape, input_dtype, channels_last: bool, bit_length: int,
                 lfsr_length: int, padding: Sequence[int], stride: Sequence[int], prog_load: Sequence[int],
                 bin_config: int, gen_config: int, xnor: bool):
        _require_cuda(weight, "PreparedConv")
        if weight.dim() != 4 or len(input_shape) != 4 or int(input_shape[1]) != weight.size(1):
            raise ValueError("PreparedConv: expected input shape [N,C,H,W] and weight [Co,C,KH,KW]")
        if input_dtype not in _DTYPES:
            raise ValueError("PreparedConv: activations must be float32, float16 or bfloat16")
        lib = _lib.load()
        self._dev = weight.device
        self._shape = tuple(int(v) for v in input_shape)
        self._dtype = input_dtype
        self._cl = bool(channels_last)
        with torch.cuda.device(self._dev):
            w_cl = _is_channels_last(weight)
            w = _dense(_float_kind(weight), w_cl)
            d = _lib.ScConvDesc()
            d.batch, d.c_in, d.h_in, d.w_in = self._shape
            d.c_out, _, d.kh, d.kw = w.shape
            d.pad_w, d.pad_h = int(padding[0]), int(padding[1])
            d.stride_h, d.stride_w = int(stride[0]), int(stride[1])
            d.act_dtype, d.act_channels_last = _DTYPES[input_dtype], int(self._cl)
            d.w_dtype, d.w_channels_last = _DTYPES[w.dtype], int(w_cl)
            d.out_channels_last = int(self._cl)
            d.bit_length, d.lfsr_length = int(bit_length), int(lfsr_length)
            d.bin_config, d.gen_config, d.xnor = int(bin_config), int(gen_config), int(bool(xnor))
            d.prog_total_width, d.prog_load_width, d.prog_load_wait = (int(v) for v in prog_load)
            d.linear_seeds = 0
            d.kernel = _kernel()
            nbytes = lib.rexsc_sc_conv2d_workspace_size(C.byref(d))
            if nbytes == 0:
                raise ValueError("PreparedConv: unsupported shape or configuration")
            self._d = d
            self._ws = torch.empty(nbytes, dtype=torch.uint8, device=self._dev)
            self._oh = (d.h_in + 2 * d.pad_h - d.kh) // d.stride_h + 1
            self._ow = (d.w_in + 2 * d.pad_w - d.kw) // d.stride_w + 1
            rc = lib.rexsc_sc_conv2d_expand(C.byref(d), None, _ptr(w), _ptr(self._ws), nbytes, _stream(self._dev))
            _lib.check(rc, "rexsc_sc_conv2d_expand (weights)")

    def __call__(self, input: torch.Tensor) -> List[torch.Tensor]:
        _require_cuda(input, "PreparedConv")
        fmt = torch.channels_last if self._cl else torch.contiguous_format
        if (tuple(input.shape) != self._shape or input.dtype != self._dtype or input.device != self._dev
                or not input.is_contiguous(memory_format=fmt)):
            raise ValueError("PreparedConv: the input does not match the shape, dtype, device or memory format the "
                             "object was prepared for")
        lib = _lib.load()
        d = self._d
        with torch.cuda.device(self._dev):
            pos = torch.empty((d.batch, d.c_out, self._oh, self._ow), dtype=torch.int16, device=self._dev,
                              memory_format=fmt)
            neg = torch.empty_like(pos)
            st = _stream(self._dev)
            rc = lib.rexsc_sc_conv2d_expand(C.byref(d), _ptr(input), None, _ptr(self._ws), self._ws.numel(), st)
            _lib.check(rc, "rexsc_sc_conv2d_expand (activations)")
            rc = lib.rexsc_sc_conv2d_accumulate(C.byref(d), _ptr(pos), _ptr(neg), _ptr(self._ws), self._ws.numel(), st)
            _lib.check(rc, "rexsc_sc_conv2d_accumulate")
        return [pos, neg]


@_traced
def conv2d_generic_general_acc(input, weight, bit_length, lfsr_length, z_units, padding, stride, prog_load,
                               bin_config, gen_config, xnor, mux) -> torch.Tensor:
    """SC conv2d forward, returns pos - neg as int16 (sc_cuda.cpp:73-85)."""
    pos, neg = conv2d_generic_general_split_acc(input, weight, bit_length, lfsr_length, z_units, padding, stride,
                                                prog_load, bin_config, gen_config, xnor, mux)
    return pos - neg


def workspace_status(device=None) -> int:
    """Synchronise and return the device status of the current stream's workspace (0 = OK)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = (dev.index, torch.cuda.current_stream(dev).cuda_stream)
    buf = _workspaces.get(key)
    if buf is None:
        return 0
    with torch.cuda.device(dev):
        return _lib.load().rexsc_workspace_status(_ptr(buf), _stream(dev))


@_traced
def linear_generic_general_acc(input: torch.Tensor, weight: torch.Tensor, prog_load: Sequence[int], bit_length: int,
                               lfsr_length: int, bin_config: int, gen_config: int, xnor: bool,
                               mux: bool, *, weight_seeds: Sequence[int] = (13, 13)) -> List[torch.Tensor]:
    """SC linear forward, returns [pos, neg] int16 [B, Cout] (sc_cuda.cpp:101-120).  ``xnor`` is ignored, as in
    the reference's linear generators (sc_cuda_matmul.cu:27-57).  ``weight_seeds`` (not in the reference's op): seed
    offsets of the positive / negative weight generators; (13, 13) is the extension, (67, 37) the front end's
    pure-torch bit loop (utils_functional.py:147-149)."""
    _require_cuda(input, "linear_generic_general_acc")
    _require_cuda(weight, "linear_generic_general_acc")
    if input.dim() != 2 or weight.dim() != 2 or input.size(1) != weight.size(1):
        raise ValueError("linear_generic_general_acc: expected input [B,C] and weight [Co,C]")
    lib = _lib.load()
    dev = input.device
    with torch.cuda.device(dev):
        x = _float_kind(input).contiguous()
        w = _float_kind(weight).contiguous()
        B, Cin = x.shape
        Co = w.shape[0]
        nbytes = lib.rexsc_sc_linear_workspace_size(B, Cin, Co, int(bit_length), int(lfsr_length), int(gen_config))
        if nbytes == 0:
            raise ValueError("linear_generic_general_acc: unsupported shape or configuration")
        pos = torch.empty((B, Co), dtype=torch.int16, device=dev)
        neg = torch.empty((B, Co), dtype=torch.int16, device=dev)
        ws = _workspace(dev, nbytes)
        rc = lib.rexsc_sc_linear_fwd_seeded(B, Cin, Co, _DTYPES[x.dtype], _DTYPES[w.dtype], int(bit_length),
                                            int(lfsr_length), int(bin_config), int(gen_config), int(prog_load[0]),
                                            int(prog_load[1]), int(prog_load[2]), int(weight_seeds[0]),
                                            int(weight_seeds[1]), _ptr(x), _ptr(w), _ptr(pos), _ptr(neg),
                                            _ptr(ws), ws.numel(), _stream(dev))
        _lib.check(rc, "rexsc_sc_linear_fwd_seeded")
    return [pos, neg]


# ---- point-wise ops -----------------------------------------------------------------------------------
class _NoiseState:
    """Seed and call counter of the counter-based Philox noise, per device; plain integers so that they can be
    stored in a checkpoint (the reference keeps 320000 opaque cuRAND states, sc_cuda_pw.cu:847-851)."""

    def __init__(self):
        self.seed = 0
        self.offsets: dict = {}

    def next(self, device_index: int) -> Tuple[int, int]:
        off = self.offsets.get(device_index, 0)
        self.offsets[device_index] = off + 1
        return self.seed, off


_noise = _NoiseState()


def manual_seed(seed: int, rank: int = 0) -> None:
    """Seed the error-injection noise; ``rank`` decorrelates data-parallel replicas."""
    _noise.seed = (int(seed) & 0xFFFFFFFF) | ((int(rank) & 0xFFFFFFFF) << 32)
    _noise.offsets.clear()


def get_rng_state() -> dict:
    return {"seed": _noise.seed, "offsets": dict(_noise.offsets)}


def set_rng_state(state: dict) -> None:
    _noise.seed = int(state["seed"])
    _noise.offsets = {int(k): int(v) for k, v in state["offsets"].items()}


def _check_or_n(or_n: int, what: str) -> int:
    or_n = int(or_n)
    if or_n < 1 or or_n > 4:
        raise ValueError(f"{what}: or_n must be 1..4 (got {or_n}); larger n is handled in Python by the caller")
    return or_n


def _coef(t: torch.Tensor, dev, what: str) -> torch.Tensor:
    if t.numel() < 6:
        raise ValueError(f"{what}: coefficient tensors need at least 6 entries")
    return t.to(device=dev, dtype=torch.float32).contiguous()


def _match_layout(t: torch.Tensor, like: torch.Tensor) -> torch.Tensor:
    """Return ``t`` with exactly ``like``'s strides so that flat memory order pairs the same logical elements."""
    if t.stride() == like.stride():
        return t
    out = torch.empty_like(like, dtype=t.dtype)
    out.copy_(t)
    return out


@_traced
def or_approx_n_forward_acc(input: torch.Tensor, or_n: int) -> torch.Tensor:
    """f_n(input) as float32, same strides as the input (sc_cuda_pw.cu:708-746)."""
    _require_cuda(input, "or_approx_n_forward_acc")
    or_n = _check_or_n(or_n, "or_approx_n_forward_acc")
    lib = _lib.load()
    dev = input.device
    with torch.cuda.device(dev):
        x = _flat_dense(_float_kind(input))
        out = torch.empty_like(x, dtype=torch.float32)
        _lib.check(lib.rexsc_orn_fwd(_ptr(x), _DTYPES[x.dtype], _ptr(out), x.numel(), or_n, _stream(dev)),
                   "rexsc_orn_fwd")
    return out


def _require_f32_grad(grad: torch.Tensor, what: str) -> None:
    if grad.dtype != torch.float32:
        # the reference fails the same way through data_ptr<float>() (sc_cuda_pw.cu:782,971)
        raise RuntimeError(f"{what}: expected scalar type Float for grad_output but found {grad.dtype}")


@_traced
def or_approx_n_backward_acc(grad_output: torch.Tensor, input: torch.Tensor, or_n: int) -> torch.Tensor:
    """grad_output * f_n'(fp16(input)) as float32 (sc_cuda_pw.cu:767-811)."""
    _require_cuda(grad_output, "or_approx_n_backward_acc")
    _require_f32_grad(grad_output, "or_approx_n_backward_acc")
    or_n = _check_or_n(or_n, "or_approx_n_backward_acc")
    lib = _lib.load()
    dev = grad_output.device
    with torch.cuda.device(dev):
        g = _flat_dense(grad_output)
        x = _match_layout(_float_kind(input), g)
        out = torch.empty_like(g)
        _lib.check(lib.rexsc_orn_bwd(_ptr(g), _ptr(x), _DTYPES[x.dtype], _ptr(out), g.numel(), or_n, _stream(dev)),
                   "rexsc_orn_bwd")
    return out


@_traced
def or_approx_n_forward_bias_std_both_acc(input_pos: torch.Tensor, input_neg: torch.Tensor, bias_coef: torch.Tensor,
                                          std_coef: torch.Tensor, or_n: int) -> torch.Tensor:
    """y(f_n(pos)) - y(f_n(neg)) with bias polynomial and Gaussian error injection, float32
    (sc_cuda_pw.cu:863-927)."""
    _require_cuda(input_pos, "or_approx_n_forward_bias_std_both_acc")
    or_n = _check_or_n(or_n, "or_approx_n_forward_bias_std_both_acc")
    lib = _lib.load()
    dev = input_pos.device
    with torch.cuda.device(dev):
        p = _flat_dense(_float_kind(input_pos))
        n = _match_layout(_float_kind(input_neg).to(p.dtype), p)
        b = _coef(bias_coef, dev, "or_approx_n_forward_bias_std_both_acc")
        s = _coef(std_coef, dev, "or_approx_n_forward_bias_std_both_acc")
        out = torch.empty_like(p, dtype=torch.float32)
        seed, off = _noise.next(dev.index)
        _lib.check(lib.rexsc_orn_bias_std_both_fwd(_ptr(p), _ptr(n), _DTYPES[p.dtype], _ptr(b), _ptr(s), _ptr(out),
                                                   p.numel(), or_n, seed, off, _stream(dev)),
                   "rexsc_orn_bias_std_both_fwd")
    return out


@_traced
def or_approx_n_backward_bias_std_both_acc(grad_output: torch.Tensor, input_pos: torch.Tensor,
                                           input_neg: torch.Tensor, bias_coef: torch.Tensor,
                                           or_n: int) -> List[torch.Tensor]:
    """Gradients w.r.t. pos and neg of the fused op, float32 (sc_cuda_pw.cu:952-1011)."""
    _require_cuda(grad_output, "or_approx_n_backward_bias_std_both_acc")
    _require_f32_grad(grad_output, "or_approx_n_backward_bias_std_both_acc")
    or_n = _check_or_n(or_n, "or_approx_n_backward_bias_std_both_acc")
    lib = _lib.load()
    dev = grad_output.device
    with torch.cuda.device(dev):
        g = _flat_dense(grad_output)
        p = _match_layout(_float_kind(input_pos), g)
        n = _match_layout(_float_kind(input_neg).to(p.dtype), g)
        b = _coef(bias_coef, dev, "or_approx_n_backward_bias_std_both_acc")
        gp = torch.empty_like(g)
        gn = torch.empty_like(g)
        _lib.check(lib.rexsc_orn_bias_std_both_bwd(_ptr(g), _ptr(p), _ptr(n), _DTYPES[p.dtype], _ptr(b), _ptr(gp),
                                                   _ptr(gn), g.numel(), or_n, _stream(dev)),
                   "rexsc_orn_bias_std_both_bwd")
    return [gp, gn]


@_traced
def or_approx_n_forward_bias_std_acc(input: torch.Tensor, bias_coef: torch.Tensor, std_coef: torch.Tensor,
                                     or_n: int) -> torch.Tensor:
    """Single-sided y(f_n(fp16(input))) returned as float16 (sc_cuda_pw.cu:834-861)."""
    _require_cuda(input, "or_approx_n_forward_bias_std_acc")
    or_n = _check_or_n(or_n, "or_approx_n_forward_bias_std_acc")
    lib = _lib.load()
    dev = input.device
    with torch.cuda.device(dev):
        x = _flat_dense(_float_kind(input))
        b = _coef(bias_coef, dev, "or_approx_n_forward_bias_std_acc")
        s = _coef(std_coef, dev, "or_approx_n_forward_bias_std_acc")
        out = torch.empty_like(x, dtype=torch.float16)
        seed, off = _noise.next(dev.index)
        _lib.check(lib.rexsc_orn_bias_std_fwd(_ptr(x), _DTYPES[x.dtype], _ptr(b), _ptr(s), _ptr(out), x.numel(),
                                              or_n, seed, off, _stream(dev)), "rexsc_orn_bias_std_fwd")
    return out


@_traced
def or_approx_n_backward_bias_std_acc(grad_output: torch.Tensor, input: torch.Tensor, bias_coef: torch.Tensor,
                                      or_n: int) -> torch.Tensor:
    """Single-sided backward, float32 (sc_cuda_pw.cu:929-950)."""
    _require_cuda(grad_output, "or_approx_n_backward_bias_std_acc")
    _require_f32_grad(grad_output, "or_approx_n_backward_bias_std_acc")
    or_n = _check_or_n(or_n, "or_approx_n_backward_bias_std_acc")
    lib = _lib.load()
    dev = grad_output.device
    with torch.cuda.device(dev):
        g = _flat_dense(grad_output)
        x = _match_layout(_float_kind(input), g)
        b = _coef(bias_coef, dev, "or_approx_n_backward_bias_std_acc")
        out = torch.empty_like(g)
        _lib.check(lib.rexsc_orn_bias_std_bwd(_ptr(g), _ptr(x), _DTYPES[x.dtype], _ptr(b), _ptr(out), g.numel(),
                                              or_n, _stream(dev)), "rexsc_orn_bias_std_bwd")
    return out


# ---- caller arithmetic on the SC counts (one pass each) ------------------------------------------------------
@_traced
def sc_counts_to_value(result_pos: torch.Tensor, result_neg: torch.Tensor, bit_length: int,
                       dtype: torch.dtype = torch.float32, split: bool = True, diff: bool = False):
    """``result.to(dtype) / bit_length`` for both signs and, with ``diff``, their difference, in one pass over the
    int16 counts instead of the caller's two casts, two divisions and subtraction
    (utils_functional.py:1181-1182,1273-1274,1324).  Bit-identical to that eager sequence.  Returns
    ``(val_pos, val_neg)``, ``val_diff`` or ``(val_pos, val_neg, val_diff)`` with the strides of ``result_pos``."""
    _require_cuda(result_pos, "sc_counts_to_value")
    _require_cuda(result_neg, "sc_counts_to_value")
    if result_pos.dtype != torch.int16 or result_neg.dtype != torch.int16:
        raise ValueError("sc_counts_to_value: counts must be the int16 tensors the SC conv returns")
    if result_pos.shape != result_neg.shape:
        raise ValueError("sc_counts_to_value: pos and neg differ in shape")
    if dtype not in (torch.float32, torch.float16):
        raise ValueError("sc_counts_to_value: dtype must be float32 or float16")
    if not (split or diff):
        raise ValueError("sc_counts_to_value: nothing to compute")
    lib = _lib.load()
    dev = result_pos.device
    with torch.cuda.device(dev):
        p = _flat_dense(result_pos)
        n = _match_layout(result_neg, p)
        vp = torch.empty_like(p, dtype=dtype) if split else None
        vn = torch.empty_like(p, dtype=dtype) if split else None
        vd = torch.empty_like(p, dtype=dtype) if diff else None
        null = C.c_void_p(0)
        _lib.check(lib.rexsc_sc_counts_to_value(_ptr(p), _ptr(n), int(bit_length), _DTYPES[dtype],
                                                _ptr(vp) if split else null, _ptr(vn) if split else null,
                                                _ptr(vd) if diff else null, p.numel(), _stream(dev)),
                   "rexsc_sc_counts_to_value")
    if split and diff:
        return vp, vn, vd
    return (vp, vn) if split else vd


CALIB_BINS = 30


def _calib_operands(result_pos, result_neg, value_pos, value_neg, what):
    for t in (result_pos, result_neg, value_pos, value_neg):
        _require_cuda(t, what)
    if result_pos.dtype != torch.int16 or result_neg.dtype != torch.int16:
        raise ValueError(f"{what}: counts must be int16")
    if not (result_pos.shape == result_neg.shape == value_pos.shape == value_neg.shape):
        raise ValueError(f"{what}: counts and values differ in shape")
    p = _flat_dense(result_pos)
    n = _match_layout(result_neg, p)
    gdt = torch.float16 if value_pos.dtype == torch.float16 and value_neg.dtype == torch.float16 else torch.float32
    gp = _match_layout(value_pos.detach().to(gdt), p)
    gn = _match_layout(value_neg.detach().to(gdt), p)
    return p, n, gp, gn, gdt


@_traced
def sc_calib_stats(result_pos: torch.Tensor, result_neg: torch.Tensor, value_pos: torch.Tensor,
                   value_neg: torch.Tensor, bit_length: int, counts_via_half: bool = False,
                   between=None) -> torch.Tensor:
    """Per-window statistics of ``err = counts / bit_length - value`` for the calibration fit, computed on the
    device without a host synchronisation (replaces the masked passes of compute_bias_std_coef,
    utils_functional.py:917-925).  Returns a float64 CUDA tensor of 91 entries: ``[:90].view(30, 3)`` are
    ``(count, sum err, sum err^2)`` of the windows ``[e_i, e_i + 0.1)``, ``e = linspace(0, max(counts)/L, 30)``;
    the first 4 bytes of entry 90 hold the largest count as int32.

    Half-precision guide values are widened to float32 before the window comparisons and the subtraction (the result
    equals the reference function on ``a_act.float()``); the reference's front end always passes float32 guides.

    ``between(stats)``, if given, runs after the maximum is known and before the windows are filled: a batch
    sharded over several GPUs all-reduces the maximum there (``sharding.reduce_calib_max_``) so that all ranks use
    the same windows."""
    p, n, gp, gn, gdt = _calib_operands(result_pos, result_neg, value_pos, value_neg, "sc_calib_stats")
    lib = _lib.load()
    dev = p.device
    with torch.cuda.device(dev):
        stats = torch.empty((CALIB_BINS * 3 + 1,), dtype=torch.float64, device=dev)
        if between is None:
            _lib.check(lib.rexsc_sc_calib_stats(_ptr(p), _ptr(n), _ptr(gp), _ptr(gn), _DTYPES[gdt], int(bit_length),
                                                1 if counts_via_half else 0, p.numel(), _ptr(stats), _stream(dev)),
                       "rexsc_sc_calib_stats")
        else:
            _lib.check(lib.rexsc_sc_calib_max(_ptr(p), _ptr(n), int(bit_length), p.numel(), _ptr(stats),
                                              _stream(dev)), "rexsc_sc_calib_max")
            between(stats)
            _lib.check(lib.rexsc_sc_calib_windows(_ptr(p), _ptr(n), _ptr(gp), _ptr(gn), _DTYPES[gdt],
                                                  int(bit_length), 1 if counts_via_half else 0, p.numel(),
                                                  _ptr(stats), _stream(dev)), "rexsc_sc_calib_windows")
    return stats


def fit_bias_std_coef(stats: torch.Tensor, bit_length: int, order: int = 5, counts_via_half: bool = False,
                      device=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """The host half of the calibration: window sums (the 91-entry block of :func:`sc_calib_stats`, on any device)
    -> per-window mean / unbiased std of err -> least-squares polynomials over the window starts, with the rules of
    compute_bias_std_coef (utils_functional.py:919-950): windows with fewer than two elements are left out, the
    bias fit is skipped (zeros) when ``order >= valid_windows // 5``.  Needs no GPU."""
    import numpy as np
    dev = torch.device(device) if device is not None else stats.device
    raw = stats.detach().cpu().contiguous()
    max_count = int(raw[CALIB_BINS * 3:].view(torch.int32)[0])
    top = float(torch.tensor(max_count, dtype=torch.float16 if counts_via_half else torch.float32)) / bit_length
    sums = raw[:CALIB_BINS * 3].view(CALIB_BINS, 3).numpy()
    output_range = np.linspace(0, top, CALIB_BINS)
    valid = sums[:, 0] > 1
    cnt = sums[valid, 0]
    mean = sums[valid, 1] / cnt
    var = np.maximum(sums[valid, 2] - cnt * mean * mean, 0.0) / (cnt - 1)
    bias_bins = torch.tensor(mean, dtype=torch.float32, device=dev)
    std_bins = torch.tensor(np.sqrt(var), dtype=torch.float32, device=dev)
    output_range = output_range[valid]
    basis = torch.from_numpy(np.stack([output_range ** i for i in range(order + 1)], axis=1)).to(dev).float()
    if order >= int(valid.sum()) // 5:
        bias_coef = torch.zeros(order + 1, device=dev)
    else:
        bias_coef = torch.linalg.lstsq(basis, bias_bins)[0]
    std_coef = torch.linalg.lstsq(basis, std_bins)[0]
    return bias_coef, std_coef


def compute_bias_std_coef(or_n: int, result_pos: torch.Tensor, result_neg: torch.Tensor, value_pos: torch.Tensor,
                          value_neg: torch.Tensor, bit_length: int, order: int = 5,
                          counts_via_half: bool = False, across_ranks: bool = False
                          ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Calibration fit with the same result as compute_bias_std_coef (utils_functional.py:901-950) called on
    ``cat(pos, neg) / bit_length`` and ``cat(value_pos, value_neg)``, taking the int16 counts and the guide values
    directly.  The window statistics come from one device pass (:func:`sc_calib_stats`) and one 728-byte read-back;
    the two least-squares fits run in torch, as there (:func:`fit_bias_std_coef`).

    ``across_ranks=True`` (inside an initialised torch.distributed job) calibrates on the global batch instead of
    this rank's shard: the maximum count and then the window sums are all-reduced, 728 bytes in all, so every rank
    fits identical coefficients and the replicas cannot drift apart."""
    dev = result_pos.device
    if or_n < 0:
        return torch.zeros(order + 1, device=dev), torch.zeros(order + 1, device=dev)
    if across_ranks:
        from . import sharding
        stats = sc_calib_stats(result_pos, result_neg, value_pos, value_neg, bit_length, counts_via_half,
                               between=sharding.reduce_calib_max_)
        sharding.reduce_calib_sums_(stats)
    else:
        stats = sc_calib_stats(result_pos, result_neg, value_pos, value_neg, bit_length, counts_via_half)
    return fit_bias_std_coef(stats, bit_length, order, counts_via_half, dev)


# ---- FXP conv -------------------------------------------------------------------------------------------
@_traced
def conv2d_saturate_acc(input: torch.Tensor, weight: torch.Tensor, add_config: int, precision_in: int,
                        precision_out: int, padding: Sequence[int], stride: Sequence[int]) -> torch.Tensor:
    """FXP saturating conv forward, int32 NCHW (fixed_cuda.cpp:24-34)."""
    _require_cuda(input, "conv2d_saturate_acc")
    _require_cuda(weight, "conv2d_saturate_acc")
    if input.dim() != 4 or weight.dim() != 4 or input.size(1) != weight.size(1):
        raise ValueError("conv2d_saturate_acc: expected input [N,C,H,W] and weight [Co,C,KH,KW]")
    lib = _lib.load()
    dev = input.device
    with torch.cuda.device(dev):
        # the reference kernel indexes both tensors as dense NCHW (fixed_cuda_kernel.cu:125,179-182)
        x = _float_kind(input).contiguous()
        w = _float_kind(weight).contiguous()
        d = _lib.FxpConvDesc()
        d.batch, d.c_in, d.h_in, d.w_in = x.shape
        d.c_out, _, d.kh, d.kw = w.shape
        d.pad_w, d.pad_h = int(padding[0]), int(padding[1])
        d.stride_h, d.stride_w = int(stride[0]), int(stride[1])
        d.act_dtype, d.w_dtype = _DTYPES[x.dtype], _DTYPES[w.dtype]
        d.add_config, d.precision_in, d.precision_out = int(add_config), int(precision_in), int(precision_out)
        d.kernel = getattr(_kernel_choice, "fxp", 0)
        nbytes = lib.rexsc_fxp_conv2d_workspace_size(C.byref(d))
        if nbytes == 0:
            raise ValueError("conv2d_saturate_acc: unsupported shape or configuration")
        oh = (d.h_in + 2 * d.pad_h - d.kh) // d.stride_h + 1
        ow = (d.w_in + 2 * d.pad_w - d.kw) // d.stride_w + 1
        out = torch.empty((d.batch, d.c_out, oh, ow), dtype=torch.int32, device=dev)
        ws = _workspace(dev, nbytes)
        _lib.check(lib.rexsc_fxp_conv2d_fwd(C.byref(d), _ptr(x), _ptr(w), _ptr(out), _ptr(ws), ws.numel(),
                                            _stream(dev)), "rexsc_fxp_conv2d_fwd")
    return out


# ---- helpers used by tests and the benchmark ------------------------------------------------------------
def build_lfsr_lut(lfsr_length: int, bit_length: int, gen_config: int = 1, xnor: bool = True,
                   prog_load: Sequence[int] = (7, 8, 1), is_weight: bool = False, device="cuda") -> torch.Tensor:
    """Stream words of every (phase, value): tensor [2^l - 1, 2^l, words] of int32 bit patterns."""
    lib = _lib.load()
    dev = torch.device(device)
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    words = (bit_length * gen_config + 31) // 32
    with torch.cuda.device(dev):
        out = torch.zeros(((1 << lfsr_length) - 1, 1 << lfsr_length, words), dtype=torch.int32, device=dev)
        _lib.check(lib.rexsc_build_lfsr_lut(int(lfsr_length), int(bit_length), int(gen_config), int(bool(xnor)),
                                            int(prog_load[0]), int(prog_load[1]), int(prog_load[2]),
                                            int(bool(is_weight)), _ptr(out), _stream(dev)), "rexsc_build_lfsr_lut")
    return out


def alu_probe(blocks: int, iters: int, device="cuda") -> torch.Tensor:
    """Launch the register-only LOP3 probe; returns the sink tensor (blocks*256 words)."""
    lib = _lib.load()
    dev = torch.device(device)
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    with torch.cuda.device(dev):
        sink = torch.empty(blocks * 256, dtype=torch.int32, device=dev)
        _lib.check(lib.rexsc_alu_probe(int(blocks), int(iters), _ptr(sink), _stream(dev)), "rexsc_alu_probe")
    return sink


def mma_probe(blocks: int, iters: int, n_cols: int = 128, device="cuda") -> torch.Tensor:
    """Launch the int8 tensor-pipe probe; returns the sink tensor (blocks*128 words)."""
    lib = _lib.load()
    dev = torch.device(device)
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    with torch.cuda.device(dev):
        sink = torch.empty(blocks * 128, dtype=torch.int32, device=dev)
        _lib.check(lib.rexsc_mma_probe(int(blocks), int(iters), int(n_cols), _ptr(sink), _stream(dev)), "rexsc_mma_probe")
    return sink
