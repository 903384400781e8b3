"""ctypes binding of librexsc_b200.so.  There is no fallback: if the CUDA library is missing the
import of any op fails loudly (build it with ``python -m rexsc_b200.build``)."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "librexsc_b200.so")

OK = 0
ERRORS = {
    -1: "REXSC_E_BAD_ARG", -2: "REXSC_E_UNSUPPORTED", -3: "REXSC_E_WORKSPACE", -4: "REXSC_E_TOO_LONG",
    -5: "REXSC_E_CUDA", -6: "REXSC_E_DEVICE_TIMEOUT", -7: "REXSC_E_STATIC_SCRATCH",
}
F32, F16, BF16 = 0, 1, 2
KERNEL_AUTO, KERNEL_DIRECT, KERNEL_TILED, KERNEL_TENSOR = 0, 1, 2, 3


class ScConvDesc(C.Structure):
    """Mirror of rexsc_sc_conv_desc (include/rexsc_b200.h)."""
    _fields_ = [(n, C.c_int32) for n in (
        "batch", "c_in", "h_in", "w_in", "c_out", "kh", "kw", "pad_h", "pad_w", "stride_h", "stride_w",
        "act_dtype", "act_channels_last", "w_dtype", "w_channels_last", "out_channels_last",
        "bit_length", "lfsr_length", "bin_config", "gen_config", "xnor",
        "prog_total_width", "prog_load_width", "prog_load_wait", "linear_seeds", "kernel")]


class FxpConvDesc(C.Structure):
    """Mirror of rexsc_fxp_conv_desc (include/rexsc_b200.h)."""
    _fields_ = [(n, C.c_int32) for n in (
        "batch", "c_in", "h_in", "w_in", "c_out", "kh", "kw", "pad_h", "pad_w", "stride_h", "stride_w",
        "act_dtype", "w_dtype", "add_config", "precision_in", "precision_out", "kernel")]


# name -> (restype, argtypes); every symbol include/rexsc_b200.h declares
_vp, _i32, _i64, _u64, _sz = C.c_void_p, C.c_int32, C.c_int64, C.c_uint64, C.c_size_t
SYMBOLS = {
    "rexsc_abi_version": (C.c_int, []),
    "rexsc_last_cuda_error": (C.c_char_p, []),
    "rexsc_kernel_launch_count": (C.c_ulonglong, []),
    "rexsc_sc_conv2d_workspace_size": (_sz, [C.POINTER(ScConvDesc)]),
    "rexsc_sc_conv2d_kernel_choice": (C.c_int, [C.POINTER(ScConvDesc)]),
    "rexsc_sc_conv2d_fwd": (C.c_int, [C.POINTER(ScConvDesc), _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "rexsc_sc_conv2d_static_scratch_bytes": (_sz, []),
    "rexsc_sc_conv2d_fwd_static": (C.c_int, [C.POINTER(ScConvDesc), _vp, _vp, _vp, _vp, _vp]),
    "rexsc_sc_conv2d_static_status": (C.c_int, [_vp]),
    "rexsc_sc_conv2d_expand": (C.c_int, [C.POINTER(ScConvDesc), _vp, _vp, _vp, _sz, _vp]),
    "rexsc_sc_conv2d_accumulate": (C.c_int, [C.POINTER(ScConvDesc), _vp, _vp, _vp, _sz, _vp]),
    "rexsc_sc_linear_workspace_size": (_sz, [_i32] * 6),
    "rexsc_sc_linear_fwd": (C.c_int, [_i32] * 12 + [_vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "rexsc_sc_linear_fwd_seeded": (C.c_int, [_i32] * 14 + [_vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "rexsc_workspace_status": (C.c_int, [_vp, _vp]),
    "rexsc_build_lfsr_lut": (C.c_int, [_i32] * 8 + [_vp, _vp]),
    "rexsc_orn_fwd": (C.c_int, [_vp, _i32, _vp, _i64, _i32, _vp]),
    "rexsc_orn_bwd": (C.c_int, [_vp, _vp, _i32, _vp, _i64, _i32, _vp]),
    "rexsc_orn_bias_std_both_fwd": (C.c_int, [_vp, _vp, _i32, _vp, _vp, _vp, _i64, _i32, _u64, _u64, _vp]),
    "rexsc_orn_bias_std_both_bwd": (C.c_int, [_vp, _vp, _vp, _i32, _vp, _vp, _vp, _i64, _i32, _vp]),
    "rexsc_orn_bias_std_fwd": (C.c_int, [_vp, _i32, _vp, _vp, _vp, _i64, _i32, _u64, _u64, _vp]),
    "rexsc_orn_bias_std_bwd": (C.c_int, [_vp, _vp, _i32, _vp, _vp, _i64, _i32, _vp]),
    "rexsc_sc_counts_to_value": (C.c_int, [_vp, _vp, _i32, _i32, _vp, _vp, _vp, _i64, _vp]),
    "rexsc_sc_calib_stats": (C.c_int, [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i64, _vp, _vp]),
    "rexsc_sc_calib_max": (C.c_int, [_vp, _vp, _i32, _i64, _vp, _vp]),
    "rexsc_sc_calib_windows": (C.c_int, [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i64, _vp, _vp]),
    "rexsc_fxp_conv2d_workspace_size": (_sz, [C.POINTER(FxpConvDesc)]),
    "rexsc_fxp_conv2d_fwd": (C.c_int, [C.POINTER(FxpConvDesc), _vp, _vp, _vp, _vp, _sz, _vp]),
    "rexsc_alu_probe": (C.c_int, [_i32, _i32, _vp, _vp]),
    "rexsc_mma_probe": (C.c_int, [_i32, _i32, _i32, _vp, _vp]),
}

_lib = None


def load() -> C.CDLL:
    """Load the CUDA library and bind every declared symbol; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: the rexsc_b200 ops have no CPU or PyTorch fallback. "
            "Build the CUDA library first:  python -m rexsc_b200.build")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SYMBOLS.items():
        fn = getattr(lib, name)  # AttributeError if the header and the library disagree
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(rc: int, what: str) -> None:
    if rc == OK:
        return
    name = ERRORS.get(rc, str(rc))
    detail = ""
    if rc == -5:
        detail = ": " + (load().rexsc_last_cuda_error() or b"").decode(errors="replace")
    if rc in (-1, -2, -4):
        raise ValueError(f"{what}: {name}{detail}")
    raise RuntimeError(f"{what}: {name}{detail}")
