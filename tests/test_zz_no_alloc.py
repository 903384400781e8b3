"""The allocation-free SC conv entry point (rexsc_sc_conv2d_fwd_static) against the ordinary one.

Some callers of the library are not allowed to allocate device memory -- a plugin whose host application has
given all device memory to its own pool, or a running loop that bans cudaMalloc/cudaFree because they
synchronise the device -- so one entry point takes its scratch from a fixed array inside the library.  This
file checks, through the C ABI, that it returns exactly what rexsc_sc_conv2d_fwd returns (integer outputs:
bit-exact) on two calls in a row that share the array, and that a call too large for the array is refused.
It is collected last so that a failure here cannot hide another test's result."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _desc(lib_mod, x, w, stride, or_n, bit_length):
    d = lib_mod.ScConvDesc()
    d.batch, d.c_in, d.h_in, d.w_in = x.shape
    d.c_out, _, d.kh, d.kw = w.shape
    d.pad_h = d.pad_w = 1
    d.stride_h = d.stride_w = stride
    d.act_dtype, d.act_channels_last, d.w_dtype, d.w_channels_last, d.out_channels_last = 0, 1, 0, 1, 1
    d.bit_length, d.lfsr_length, d.bin_config, d.gen_config, d.xnor = bit_length, -1, or_n - 1, 1, 1
    d.prog_total_width, d.prog_load_width, d.prog_load_wait = 7, 8, 1
    return d


def _run_both(lib_mod, lib, case, seed):
    N, Cin, H, Cout, stride, or_n, L = case
    g = torch.Generator().manual_seed(seed)
    dev = torch.device("cuda", 0)
    x = torch.rand(N, Cin, H, H, generator=g).to(dev).contiguous(memory_format=torch.channels_last)
    w = (torch.randn(Cout, Cin, 3, 3, generator=g) * 0.1).clamp(-1, 1).to(dev).contiguous(
        memory_format=torch.channels_last)
    d = _desc(lib_mod, x, w, stride, or_n, L)
    oh = (H + 2 - 3) // stride + 1
    outs = [torch.full((N, Cout, oh, oh), -7, dtype=torch.int16, device=dev).contiguous(
        memory_format=torch.channels_last) for _ in range(4)]
    st = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    vp = lambda t: C.c_void_p(t.data_ptr())
    nbytes = lib.rexsc_sc_conv2d_workspace_size(C.byref(d))
    assert 0 < nbytes <= lib.rexsc_sc_conv2d_static_scratch_bytes()
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    rc = lib.rexsc_sc_conv2d_fwd(C.byref(d), vp(x), vp(w), vp(outs[0]), vp(outs[1]), vp(ws), nbytes, st)
    assert rc == 0
    rc = lib.rexsc_sc_conv2d_fwd_static(C.byref(d), vp(x), vp(w), vp(outs[2]), vp(outs[3]), st)
    assert rc == 0, rc
    torch.cuda.synchronize()
    assert lib.rexsc_sc_conv2d_static_status(st) == 0    # no bounded device wait gave up in the static call
    assert int(outs[0].min()) >= 0                       # the sentinel was overwritten everywhere
    assert torch.equal(outs[2], outs[0]), f"{case}: pos differs from the workspace entry point"
    assert torch.equal(outs[3], outs[1]), f"{case}: neg differs from the workspace entry point"


def test_static_scratch_entry_point_matches_workspace_entry_point():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from rexsc_b200 import _lib as lib_mod

    lib = lib_mod.load()
    torch.cuda.set_device(0)
    # two calls in a row on the shared array; the second is smaller and of another configuration, so anything
    # the first left behind (longer tables, more words, other signs) would show if it leaked into a result
    _run_both(lib_mod, lib, (4, 64, 20, 48, 1, 2, 64), seed=1)
    _run_both(lib_mod, lib, (2, 24, 11, 40, 2, 3, 32), seed=2)
    # and the first configuration once more, after the smaller one
    _run_both(lib_mod, lib, (4, 64, 20, 48, 1, 2, 64), seed=3)


def test_static_scratch_rejects_oversized_calls():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from rexsc_b200 import _lib as lib_mod

    lib = lib_mod.load()
    d = lib_mod.ScConvDesc()
    d.batch, d.c_in, d.h_in, d.w_in, d.c_out, d.kh, d.kw = 256, 64, 58, 58, 64, 3, 3
    d.stride_h = d.stride_w = 1
    d.bit_length, d.lfsr_length, d.bin_config, d.gen_config = 32, -1, 1, 1
    d.prog_total_width, d.prog_load_width, d.prog_load_wait = 7, 8, 1
    assert lib.rexsc_sc_conv2d_workspace_size(C.byref(d)) > lib.rexsc_sc_conv2d_static_scratch_bytes()
    one = C.c_void_p(256)
    assert lib.rexsc_sc_conv2d_fwd_static(C.byref(d), one, one, one, one, None) == -7
    d.bit_length = 48   # invalid stream length: the ordinary validation answers
    assert lib.rexsc_sc_conv2d_fwd_static(C.byref(d), one, one, one, one, None) == -2
