"""CPU-only checks of the C-ABI shared library: it loads, exports every symbol the public header declares,
and its host-side planning (workspace sizes, argument validation) behaves.  No kernel is launched."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "rexsc_b200.h")


@pytest.fixture(scope="module")
def lib():
    from rexsc_b200 import build, _lib

    build.build()
    return _lib.load()


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(rexsc_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound(lib):
    from rexsc_b200 import _lib

    names = declared_symbols()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/rexsc_b200.h but not exported"
        assert n in _lib.SYMBOLS, f"{n} has no ctypes prototype"
    assert set(_lib.SYMBOLS) == set(names)
    assert lib.rexsc_abi_version() == 1


def _desc(**kw):
    from rexsc_b200 import _lib

    d = _lib.ScConvDesc()
    base = dict(batch=2, c_in=8, h_in=10, w_in=10, c_out=16, kh=3, kw=3, pad_h=0, pad_w=0, stride_h=1, stride_w=1,
                bit_length=32, lfsr_length=-1, bin_config=1, gen_config=1, xnor=1, prog_total_width=7,
                prog_load_width=8, prog_load_wait=1)
    base.update(kw)
    for k, v in base.items():
        setattr(d, k, v)
    return d


def test_workspace_size_model(lib):
    d = _desc()
    n = lib.rexsc_sc_conv2d_workspace_size(C.byref(d))
    assert n > 0 and n % 256 == 0
    # activation words dominate: planes * padded channels * padded pixel count * 4 bytes
    big = _desc(batch=256, c_in=64, h_in=58, w_in=58, c_out=64)
    nb = lib.rexsc_sc_conv2d_workspace_size(C.byref(big))
    assert 256 * 58 * 58 * 64 * 4 <= nb <= 256 * 58 * 58 * 64 * 4 * 2.6   # padded row pitch + bit planes of the tensor-core kernel
    two = _desc(batch=256, c_in=64, h_in=58, w_in=58, c_out=64, bit_length=64)
    assert lib.rexsc_sc_conv2d_workspace_size(C.byref(two)) > 1.9 * nb


@pytest.mark.parametrize("bad", [dict(bit_length=48), dict(bin_config=-1), dict(c_in=0), dict(stride_h=0),
                                 dict(kh=20), dict(bit_length=256), dict(gen_config=0), dict(act_dtype=7)])
def test_bad_descriptors_are_rejected_on_the_host(lib, bad):
    d = _desc(**bad)
    assert lib.rexsc_sc_conv2d_workspace_size(C.byref(d)) == 0
    rc = lib.rexsc_sc_conv2d_fwd(C.byref(d), None, None, None, None, None, 0, None)
    assert rc < 0


def test_null_pointers_and_small_workspace(lib):
    d = _desc()
    assert lib.rexsc_sc_conv2d_fwd(C.byref(d), None, None, None, None, None, 0, None) == -1
    one = C.c_void_p(256)
    assert lib.rexsc_sc_conv2d_fwd(C.byref(d), one, one, one, one, None, 0, None) == -3
    assert lib.rexsc_sc_conv2d_fwd(C.byref(d), one, one, one, one, one, 16, None) == -3


def test_fxp_workspace_and_validation(lib):
    from rexsc_b200 import _lib

    d = _lib.FxpConvDesc()
    for k, v in dict(batch=4, c_in=3, h_in=32, w_in=32, c_out=32, kh=5, kw=5, pad_h=2, pad_w=2, stride_h=1,
                     stride_w=1, add_config=0, precision_in=5, precision_out=24).items():
        setattr(d, k, v)
    assert lib.rexsc_fxp_conv2d_workspace_size(C.byref(d)) >= 4 * 3 * 36 * 36 * 4
    d.precision_in = 0
    assert lib.rexsc_fxp_conv2d_workspace_size(C.byref(d)) == 0
    assert lib.rexsc_fxp_conv2d_fwd(C.byref(d), None, None, None, None, 0, None) < 0


def test_pointwise_argument_validation(lib):
    one = C.c_void_p(256)
    assert lib.rexsc_orn_fwd(one, 0, one, -1, 2, None) == -1
    assert lib.rexsc_orn_fwd(None, 0, one, 8, 2, None) == -1
    assert lib.rexsc_orn_fwd(one, 0, one, 0, 2, None) == 0       # empty tensor: nothing launched
    assert lib.rexsc_orn_bias_std_both_fwd(one, one, 0, None, one, one, 8, 2, 0, 0, None) == -1
    assert lib.rexsc_alu_probe(0, 1, one, None) == -1


def test_dropin_modules_expose_the_reference_names():
    import rexsc_b200

    rexsc_b200.install_dropin()
    import fixed_extension
    import fixed_extension_cuda
    import sc_extension
    import sc_extension_cuda

    for n in ("conv2d_generic_general_acc", "conv2d_generic_general_split_acc", "linear_generic_general_acc",
              "or_approx_n_forward_acc", "or_approx_n_backward_acc", "or_approx_n_forward_bias_std_acc",
              "or_approx_n_backward_bias_std_acc", "or_approx_n_forward_bias_std_both_acc",
              "or_approx_n_backward_bias_std_both_acc"):
        assert callable(getattr(sc_extension_cuda, n))
    assert callable(fixed_extension_cuda.conv2d_saturate_acc)
    with pytest.raises(NotImplementedError):
        sc_extension.conv2d_generic_general()
    with pytest.raises(NotImplementedError):
        fixed_extension.conv2d_saturate()


def test_ops_refuse_cpu_tensors():
    import torch

    from rexsc_b200 import ops

    with pytest.raises(RuntimeError):
        ops.or_approx_n_forward_acc(torch.zeros(4), 2)
    with pytest.raises(RuntimeError):
        ops.conv2d_saturate_acc(torch.zeros(1, 1, 4, 4), torch.zeros(1, 1, 3, 3), 0, 5, 24, (0, 0), (1, 1))
