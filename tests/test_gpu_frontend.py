"""The reference's UNCHANGED front end running on the drop-in ops, on a GPU, against the same front end running on
the reference's own GPU extensions (oracle/_ref, compiled unchanged for sm_100).  Layers, models and the training
loop are the reference's code (imported from a checkout or from its byte-compiled copy); this file only feeds them.

Bars: integer-derived forward values bit-identical (SC counts and FXP sums overwrite the float graph's values);
calibrated forward with zero std coefficients bit-identical; gradients within 1e-3 relative."""
import copy
import os

import pytest
import torch

from helpers import ops_of, reference_gpu_modules, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def fe(ops):
    from rexsc_b200 import frontend

    try:
        return frontend.load()
    except ImportError as exc:
        pytest.skip(str(exc))


@pytest.fixture(scope="module")
def ref_mods(ops):
    mods = reference_gpu_modules()
    if mods is None:
        pytest.skip("oracle/_ref holds no loadable reference GPU extension (python oracle/build_ref.py --gpu)")
    return mods


def _layer_run(fe, layer, x, sync, autocast):
    torch.manual_seed(1234)      # the sync=2 path draws torch.randn_like noise (utils_functional.py:441-447)
    layer.zero_grad()
    x = x.clone().requires_grad_(True)
    layer.run_args["sync"] = sync
    with torch.autocast("cuda", dtype=torch.float16, enabled=autocast):
        out = layer(x)
    # a fixed, non-trivial cotangent with the strides of the output, as the layers behind an SC conv produce it (the
    # reference's point-wise backward kernels pair gradient and saved sum by memory offset, sc_cuda_pw.cu:767-811)
    w = torch.empty_like(out, dtype=torch.float32).copy_(torch.linspace(-1, 1, out.numel(), device=out.device)
                                                          .view(out.shape))
    out.backward(w.to(out.dtype))
    return out.detach(), x.grad.detach(), layer.weight.grad.detach().clone(), layer.bias_coef.clone(), \
        layer.std_coef.clone()


@pytest.mark.parametrize("autocast", [False, True])
@pytest.mark.parametrize("channels_last", [False, True])
@pytest.mark.parametrize("sync", [1, 2, 3])
def test_conv2d_add_partial_layer(fe, ref_mods, sync, channels_last, autocast):
    """Conv2d_Add_Partial.forward (utils_class.py:41-86) -> conv2d_generic (utils_functional.py:1083-1317),
    forward + backward, in the three sync modes."""
    torch.manual_seed(10 * sync + 2 * channels_last + autocast)
    layer = fe.utils_class.Conv2d_Add_Partial(64, 48, 3, padding=1, stride=1, bias=False, forward="or_2", err=5,
                                              generator="lfsr", sync=sync).cuda()
    with torch.no_grad():
        layer.weight.mul_(3.0)                        # spread the counts over more of the stream length
        layer.bias_coef.copy_(torch.tensor([0.01, -0.05, 0.02, 0.003, -0.001, 0.0002]))
    x = torch.rand(8, 64, 14, 14, device="cuda")
    if channels_last:
        layer = layer.to(memory_format=torch.channels_last)
        x = x.contiguous(memory_format=torch.channels_last)
    twin = copy.deepcopy(layer)
    ours = _layer_run(fe, layer, x, sync, autocast)
    with ops_of(fe, ref_mods):
        ref = _layer_run(fe, twin, x, sync, autocast)
    if sync == 2:
        # same counts + same guide -> the same fit by the same torch code; then Bias_Correct on equal values
        assert torch.allclose(ours[3], ref[3], rtol=1e-4, atol=1e-6) and torch.allclose(ours[4], ref[4], rtol=1e-4,
                                                                                     atol=1e-6)
        assert ours[4].abs().sum() > 0
        assert torch.allclose(ours[0].float(), ref[0].float(), rtol=1e-4, atol=1e-5)
    else:
        assert torch.equal(ours[0], ref[0]), f"forward differs (sync {sync})"
    assert ours[0].dtype == ref[0].dtype and ours[0].stride() == ref[0].stride()
    assert rel_err(ours[1], ref[1]) < 1e-3
    assert rel_err(ours[2], ref[2]) < 1e-3


def test_strided_and_pointwise_sc_layers(fe, ref_mods):
    """The two other SC layer shapes of the ResNets: 3x3 stride 2 and the 1x1 stride-2 shortcut (resnet_sc.py:79-97)."""
    torch.manual_seed(5)
    for k, pad in ((3, 1), (1, 0)):
        layer = fe.utils_class.Conv2d_Add_Partial(64, 128, k, padding=pad, stride=2, bias=False, forward="or_2",
                                                  err=5).cuda().to(memory_format=torch.channels_last)
        x = torch.rand(4, 64, 28, 28, device="cuda").contiguous(memory_format=torch.channels_last)
        twin = copy.deepcopy(layer)
        ours = _layer_run(fe, layer, x, 1, True)
        with ops_of(fe, ref_mods):
            ref = _layer_run(fe, twin, x, 1, True)
        assert torch.equal(ours[0], ref[0])
        assert rel_err(ours[1], ref[1]) < 1e-3 and rel_err(ours[2], ref[2]) < 1e-3


class _Recorder:
    """Wraps an extension module and keeps what conv2d_saturate_acc returned, layer by layer."""

    def __init__(self, mod):
        self.mod, self.outs = mod, []

    def conv2d_saturate_acc(self, *args):
        out = self.mod.conv2d_saturate_acc(*args)
        self.outs.append(out.clone())
        return out


def test_tinyconv_fxp_forward_bit_exact_and_gradients(fe, ref_mods):
    """The fixed-point TinyConv (network.py:215-272, generator='fixed', 5-bit layers and a 7-bit classifier) at batch
    256 on U[0,1) inputs, seed 1: every layer's conv2d_saturate_acc output equal bit for bit, the loss gradient with
    respect to every weight and to the input within 1e-3 relative."""
    import fixed_extension_cuda as dropin_fx
    import sc_extension_cuda as dropin_sc

    torch.manual_seed(1)
    model = fe.network.CONV_tiny_add_partial(generator="fixed", sc_compute="full_bin", err=[5, 5, 5, 7], sync=1).cuda()
    with torch.no_grad():
        for m in (model.conv1, model.conv2, model.conv3, model.fc1):
            m.weight.copy_((torch.randn_like(m.weight) * 0.1).clamp_(-1, 1))
    twin = copy.deepcopy(model)
    x = torch.rand(256, 3, 32, 32, device="cuda")
    y = torch.randint(0, 10, (256,), device="cuda")
    crit = fe.utils.LabelSmoothLoss(0.1)
    runs = []
    for net, fx in ((model, dropin_fx), (twin, ref_mods[1])):
        rec = _Recorder(fx)
        xi = x.clone().requires_grad_(True)
        with ops_of(fe, (dropin_sc, rec)):
            loss = crit(net(xi), y)
        loss.backward()
        runs.append((rec.outs, float(loss), xi.grad.clone(), [p.grad.clone() for p in net.parameters()]))
    (o_a, l_a, gx_a, gw_a), (o_b, l_b, gx_b, gw_b) = runs
    assert len(o_a) == len(o_b) == 4
    for i, (a, b) in enumerate(zip(o_a, o_b)):
        assert a.dtype == torch.int32 and torch.equal(a, b), f"FXP layer {i + 1} differs"
    assert abs(l_a - l_b) <= 1e-6 * abs(l_b)
    assert rel_err(gx_a, gx_b) < 1e-3
    for a, b in zip(gw_a, gw_b):
        assert rel_err(a, b) < 1e-3


@pytest.mark.parametrize("sync", [1, 3])
def test_resnet18_forward_backward(fe, ref_mods, sync):
    """SC ResNet-18 (resnet_sc.py:342-365, OR-2, 32-bit streams, channels_last, fp16 autocast) at a small
    resolution: logits and every weight gradient on the drop-in against the reference's own GPU extensions."""
    torch.manual_seed(7)
    model = fe.resnet_sc.resnet18(pretrained=False, sc_compute="or_2", uniform=False, prec=7, err=5).cuda()
    model = model.to(memory_format=torch.channels_last)
    twin = copy.deepcopy(model)
    x = torch.randn(4, 3, 64, 64, device="cuda").clamp_(-3, 3).contiguous(memory_format=torch.channels_last)
    y = torch.randint(0, 1000, (4,), device="cuda")
    crit = fe.utils.LabelSmoothLoss(0.1)
    res = []
    for net, mods in ((model, None), (twin, ref_mods)):
        net.sync = sync
        net.train()

        def step():
            with torch.autocast("cuda", dtype=torch.float16):
                out = net(x)
            loss = crit(out.float(), y)
            loss.backward()
            return out.detach().float(), [p.grad.clone() for p in net.parameters() if p.grad is not None]

        if mods is None:
            res.append(step())
        else:
            with ops_of(fe, mods):
                res.append(step())
    (out_a, g_a), (out_b, g_b) = res
    assert torch.allclose(out_a, out_b, rtol=1e-3, atol=1e-3)
    assert len(g_a) == len(g_b) > 60
    worst = max(rel_err(a, b) for a, b in zip(g_a, g_b))
    assert worst < 1e-3, worst


def test_reference_training_loop_runs_on_the_drop_in(fe):
    """utils_own.train (utils_own.py:201-208) for a few iterations per sync mode on a small SC ResNet-18: finite
    losses, weights move, the sync=2 step fits calibration polynomials that the sync=3 steps then use."""
    from rexsc_b200.frontend import train

    wl = train.Workload("resnet18_small", "resnet18", "or_2", 5, 8, 64, 1000, "fp16", True, acc_limit=8)
    tr = train.Trainer(fe, wl, "cuda", seed=0)
    before = torch.cat([p.detach().reshape(-1).clone() for p in tr.model.parameters()])
    for sync in (1, 2, 3):
        r = tr.run(sync, 1, 2, barrier=False)
        assert r["ms"] > 0 and r["images"] == (8 if sync == 2 else 16)
    after = torch.cat([p.detach().reshape(-1) for p in tr.model.parameters()])
    assert torch.isfinite(after).all()
    # the optimizer stepped, or the GradScaler skipped the first steps on fp16 overflow and lowered its scale
    assert not torch.equal(before, after) or tr.scaler.get_scale() < 65536.0
    layers = train.sc_layers(fe, tr.model)
    assert len(layers) == 19
    assert sum(float(m.std_coef.abs().sum()) > 0 for m in layers) >= 15


@pytest.mark.parametrize("channels_last", [False, True])
def test_guide_conv_pair_matches_the_two_convolutions(ops, channels_last):
    """The opt-in single guide convolution against the reference's two (utils_functional.py:1199-1211): same values,
    same gradients with respect to activation and weight (1e-3 relative)."""
    from rexsc_b200.frontend.guide import guide_conv_pair

    torch.manual_seed(3)
    x = torch.rand(8, 64, 16, 16, device="cuda")
    w = (torch.randn(96, 64, 3, 3, device="cuda") * 0.1).clamp(-1, 1)
    if channels_last:
        x = x.contiguous(memory_format=torch.channels_last)
        w = w.contiguous(memory_format=torch.channels_last)
    cot = torch.randn(8, 96, 8, 8, device="cuda")
    res = []
    for fused in (False, True):
        xi, wi = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
        if fused:
            p, n = guide_conv_pair(xi, wi, (2, 2), (1, 1))
        else:
            p = torch.nn.functional.conv2d(xi, wi.clamp(0, 100), padding=(1, 1), stride=(2, 2))
            n = torch.nn.functional.conv2d(xi, -(wi.clamp(-100, 0)), padding=(1, 1), stride=(2, 2))
        (p * cot - 0.5 * n * cot).sum().backward()
        res.append((p.detach(), n.detach(), xi.grad, wi.grad))
    for a, b in zip(res[0], res[1]):
        assert rel_err(b, a) < 1e-3
    # and the halves feed the fused point-wise op like two separate tensors do
    bias = torch.tensor([0.01, -0.05, 0.02, 0.003, -0.001, 0.0002], device="cuda")
    zero = torch.zeros(6, device="cuda")
    a = ops.or_approx_n_forward_bias_std_both_acc(res[0][0], res[0][1], bias, zero, 2)
    b = ops.or_approx_n_forward_bias_std_both_acc(res[1][0], res[1][1], bias, zero, 2)
    assert rel_err(b, a) < 1e-3


@pytest.mark.parametrize("forward", ["full_or", "full_bin"])
@pytest.mark.parametrize("bit_length", [32, 64, 128])
def test_linear_generic_bit_loop_matches_the_sc_linear_op(fe, bit_length, forward):
    """The opt-in replacement of the per-bit torch loop of linear_generic (utils_functional.py:955-1082,
    generator='lfsr', shared generators) against that loop itself: values bit-identical, gradients identical (the
    guide expression is the same).  Inputs as Linear_Or feeds them (utils_class.py:197-207): quantised to 7 bits,
    activations in [0, 1) -- off the 1/bit_length grid for the shorter streams, which exercises the ceil rule -- and
    no magnitude above (bit_length - 1) / bit_length, where the extension's quantiser saturates and the torch loop
    does not (7-bit inputs with 128-bit streams, Linear_Or's defaults, never get there)."""
    from rexsc_b200.frontend.linear import linear_generic_sc

    uf = fe.utils_functional
    torch.manual_seed(bit_length + len(forward))
    top = (bit_length - 1) / bit_length
    # few, mostly small weights with some large ones: OR-1 must neither stay empty nor saturate on both signs
    c_in = 200 if forward == "full_bin" else 40
    x = uf.quantize(torch.rand(24, c_in, device="cuda"), prec=7).clamp(max=top)
    w = torch.randn(70, c_in, device="cuda") * 0.05
    w[:, ::7] *= 12
    w = uf.quantize(w.clamp(-1, 1), prec=7).clamp(-top, top)
    cot = torch.randn(24, 70, device="cuda")
    res = []
    for ours in (False, True):
        xi, wi = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
        if ours:
            out = linear_generic_sc(xi, wi, bit_length=bit_length, forward=forward, value_dtype=uf.compute_type)
        else:
            out = uf.linear_generic(xi, wi, bit_length=bit_length, forward=forward, generator="lfsr")
        (out.float() * cot).sum().backward()
        res.append((out.detach().float(), xi.grad.float(), wi.grad.float()))
    assert (res[0][0] != 0).float().mean() > 0.3, "trivial case"
    assert torch.equal(res[1][0], res[0][0]), f"{(res[1][0] != res[0][0]).sum().item()} values differ"
    assert rel_err(res[1][1], res[0][1]) < 1e-6 and rel_err(res[1][2], res[0][2]) < 1e-6
