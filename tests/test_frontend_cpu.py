"""CPU-only tests of the harness that runs the reference's unchanged front end: the import stand-ins, the
byte-compiled copy, the reference's own training loop on synthetic batches (ops stood in for by the oracle), and the
bucketed weight-gradient all-reduce with two gloo ranks.  Skipped when neither a reference checkout nor its
byte-compiled copy is present."""
import os
import socket
import subprocess
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _have_frontend():
    from rexsc_b200 import frontend

    return frontend.reference_root() is not None or frontend.have_compiled()


needs_frontend = pytest.mark.skipif(not _have_frontend(), reason="reference front end not available")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_stand_ins_import_and_refuse_use():
    from rexsc_b200 import frontend

    frontend._install_stubs()
    import bokeh.io
    import nvidia.dali.fn
    from nvidia.dali import pipeline_def
    from nvidia.dali.plugin.pytorch import DALIClassificationIterator, LastBatchPolicy  # noqa: F401

    @pipeline_def
    def pipe():
        return None

    if "stubs" in (bokeh.io.__file__ or ""):
        with pytest.raises(RuntimeError):
            bokeh.io.show()
    if "stubs" in (nvidia.dali.fn.__file__ or ""):
        with pytest.raises(RuntimeError):
            pipe()
        with pytest.raises(RuntimeError):
            nvidia.dali.fn.readers


_CHILD = r"""
import sys
sys.path[:0] = [{root!r}, {root!r} + "/oracle", {root!r} + "/tests"]
import torch
import oracle_ops_shim
oracle_ops_shim.install()
from rexsc_b200 import frontend
fe = frontend.load()
assert fe.sourceless == {sourceless}
torch.manual_seed(0)
m = fe.network.CONV_tiny_add_partial(generator='lfsr', sc_compute='or_2', err=[5, 5, 5, 7], sync=1)
x = torch.rand(2, 3, 32, 32)
outs = []
for sync in (1, 2, 3):
    m.sync = sync
    y = m(x)
    y.sum().backward()
    outs.append(float(y.detach().abs().sum()))
assert all(o == o and o > 0 for o in outs)
assert float(m.conv1.std_coef.abs().sum()) > 0          # the sync=2 pass fitted the calibration polynomials
print("OK", outs[0])
"""


@needs_frontend
@pytest.mark.parametrize("sourceless", [False, True])
def test_front_end_layers_run_from_checkout_and_from_compiled_copy(sourceless, oracle):
    from rexsc_b200 import frontend
    from rexsc_b200.frontend import build as fbuild

    if sourceless:
        if not fbuild.build():
            pytest.skip("no byte-compiled copy and no checkout to make one from")
    elif frontend.reference_root() is None:
        pytest.skip("no reference checkout")
    env = dict(os.environ, REXSC_FRONTEND_COMPILED="1" if sourceless else "0")
    r = subprocess.run([sys.executable, "-c", _CHILD.format(root=ROOT, sourceless=sourceless)], env=env,
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "OK" in r.stdout


def _reducer_worker(rank, world, port, out):
    from rexsc_b200 import sharding

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        model = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.Tanh(), torch.nn.Linear(16, 4),
                                    torch.nn.Linear(4, 3))
        unused = torch.nn.Parameter(torch.ones(5))          # a parameter that never gets a gradient
        model.register_parameter("unused", unused)
        red = sharding.GradAllReducer(model, bucket_bytes=300)   # several small buckets
        g = torch.Generator().manual_seed(100 + rank)
        grads = []
        for it in range(2):                                  # two backward passes, gradients accumulate
            x = torch.randn(6, 8, generator=g)
            model(x).square().sum().backward()
            grads.append([None if p.grad is None else p.grad.clone() for p in model.parameters()])
        out.put((rank, len(red.buckets), red.nbytes, [[None if t is None else t.tolist() for t in gs] for gs in grads]))
    finally:
        dist.destroy_process_group()


def test_bucketed_gradient_allreduce_two_gloo_ranks():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_reducer_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert results[0][1] > 1 and results[0][1:3] == results[1][1:3]
    assert results[0][3] == results[1][3]                    # identical gradients on both ranks after each backward
    # and they are the mean of what each rank would have computed alone
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.Tanh(), torch.nn.Linear(16, 4), torch.nn.Linear(4, 3))
    acc = [torch.zeros_like(p) for p in model.parameters()]
    gens = [torch.Generator().manual_seed(100 + r) for r in range(world)]
    for it in range(2):
        for r in range(world):
            model.zero_grad()
            model(torch.randn(6, 8, generator=gens[r])).square().sum().backward()
            for a, p in zip(acc, model.parameters()):
                a += p.grad / world
        got = results[0][3][it]
        assert got[0] is None                                # the unused parameter (registered on the container,
        for a, t in zip(acc, got[1:]):                       # hence listed first) still has no gradient
            assert torch.allclose(a, torch.tensor(t), rtol=1e-5, atol=1e-6)


def _train_worker(rank, world, port, out):
    sys.path[:0] = [ROOT, os.path.join(ROOT, "oracle"), os.path.join(ROOT, "tests")]
    import oracle_ops_shim

    oracle_ops_shim.install()
    from rexsc_b200 import frontend
    from rexsc_b200.frontend import train

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        fe = frontend.load()
        wl = train.Workload("tiny_or2", "tinyconv", "or_2", [5, 5, 5, 7], 4, 32, 10, "fp32", False, inputs="cifar", acc_limit=4)
        tr = train.Trainer(fe, wl, "cpu", seed=3, rank=rank, lr=1e-2)
        res = {s: tr.run(s, 1, 2, barrier=True) for s in (3, 2, 1)}
        params = torch.cat([p.detach().reshape(-1) for p in tr.model.parameters()])
        coefs = torch.cat([torch.cat([m.bias_coef, m.std_coef]) for m in train.sc_layers(fe, tr.model)])
        blended = train.blended_rate(res[1], res[2], res[3], 5000)
        out.put((rank, params.tolist(), coefs.tolist(), {k: v["images"] for k, v in res.items()}, blended,
                 tr.reducer.nbytes))
    finally:
        dist.destroy_process_group()


@needs_frontend
def test_reference_training_loop_two_gloo_ranks(oracle):
    """utils_own.train on synthetic batches, two ranks with different data: after sync 3, 2 and 1 steps the replicas
    hold identical weights (gradient all-reduce) and identical calibration coefficients (averaged after sync 2)."""
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_train_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=600) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    (_, p0, c0, im0, b0, nb0), (_, p1, c1, im1, b1, nb1) = results
    assert p0 == p1, "replicas drifted apart: weight gradients were not reduced identically"
    assert c0 == c1 and any(abs(v) > 0 for v in c0)
    assert im0 == {3: 8, 2: 4, 1: 8} == im1                 # half batch on the calibration step
    assert b0 > 0 and b1 > 0 and nb0 == nb1 > 0
    # the weights moved away from their common initial values
    torch.manual_seed(3)
    assert len(p0) > 1000
