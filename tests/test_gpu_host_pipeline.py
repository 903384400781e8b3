"""The host-buffer pipeline must return exactly what the plain op returns on device copies, for a sequence of
calls that reuses staging buffers (more calls than slots, repeated and differing shapes)."""
import pytest
import torch

from helpers import conv_inputs

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("chunks", [1, 3])
def test_pipeline_matches_plain_op(ops, chunks):
    """chunks = 3 runs every call as up to three calls on slices of its batch (uneven: 4 -> 1 + 1 + 2 images)."""
    from rexsc_b200.host_pipeline import HostConvCall, HostConvPipeline

    dev = torch.device("cuda", 0)
    shapes = [(4, 16, 12, 12, 24, 3, 1), (4, 16, 12, 12, 24, 3, 1), (2, 24, 9, 9, 40, 3, 2),
              (4, 16, 12, 12, 24, 3, 1), (2, 24, 9, 9, 40, 3, 2), (4, 16, 12, 12, 24, 3, 1)]
    calls, expect = [], []
    for i, (N, C, H, W, Co, K, s) in enumerate(shapes):
        x, w = conv_inputs(N, C, H, W, Co, K, seed=100 + i)
        x = torch.nn.functional.pad(x, (1, 1, 1, 1)).contiguous(memory_format=torch.channels_last).pin_memory()
        wd = w.to(dev).contiguous(memory_format=torch.channels_last)
        p, n = ops.conv2d_generic_general_split_acc(x.to(dev), wd, 32, -1, 16, (0, 0), (s, s), (7, 8, 1), 1, 1, True,
                                                    False)
        hp = torch.empty(p.shape, dtype=torch.int16).contiguous(memory_format=torch.channels_last).pin_memory()
        hn = torch.empty_like(hp).pin_memory()
        calls.append(HostConvCall(x, wd, hp, hn, 32, (s, s), 1))
        expect.append((p.cpu(), n.cpu()))
    pipe = HostConvPipeline(dev, chunks=chunks)
    for _ in range(2):          # second round reuses every staging buffer
        for c in calls:
            c.out_pos_host.fill_(-1)
            c.out_neg_host.fill_(-1)
        pipe.run(calls)
        torch.cuda.synchronize()
        for c, (p, n) in zip(calls, expect):
            assert torch.equal(c.out_pos_host, p) and torch.equal(c.out_neg_host, n)


def test_out_argument_is_validated(ops):
    x = torch.rand(1, 8, 6, 6).cuda()
    w = torch.rand(4, 8, 3, 3).cuda()
    bad = torch.empty(1, 4, 4, 4, dtype=torch.int32).cuda()
    with pytest.raises(ValueError):
        ops.conv2d_generic_general_split_acc(x, w, 32, -1, 16, (0, 0), (1, 1), (7, 8, 1), 0, 1, True, False,
                                             out=(bad, bad))
