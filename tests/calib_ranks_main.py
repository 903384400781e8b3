"""Rank program of tests/test_gpu_multi_rank_calib.py (started by torch.distributed.run, one rank per GPU, NCCL):
calibration over a batch sharded across the ranks.  Every rank must end with the window statistics of the whole
batch (checked against the oracle) and with coefficients identical to every other rank's."""
import os, sys, torch, torch.distributed as dist, numpy as np
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT); sys.path.insert(0, os.path.join(ROOT, 'oracle'))
from rexsc_b200 import ops, sharding
import oracle
rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
dist.init_process_group("nccl")
g = torch.Generator().manual_seed(5)
n = 400_000; L = 32
act = torch.rand(2, n, generator=g) ** 2 * 1.9
cnt = torch.round((act * (1 - 0.04 * act) + 0.04 * torch.randn(2, n, generator=g)) * L).clamp(0, 2 * L).to(torch.int16)
cnt[0, 0] = 2 * L
s, c = sharding.shard_range(n, world, rank)
sl = slice(s, s + c)
args = (cnt[0, sl].cuda(), cnt[1, sl].cuda(), act[0, sl].cuda(), act[1, sl].cuda(), L)
st = ops.sc_calib_stats(*args, between=sharding.reduce_calib_max_)
sharding.reduce_calib_sums_(st)
bias, std = ops.compute_bias_std_coef(2, *args, 5, across_ranks=True)
whole = oracle.calib_window_sums(cnt.reshape(-1).numpy() / np.float32(L), act.reshape(-1).numpy())
got = st[:90].cpu().view(30, 3).numpy()
ok = np.array_equal(got[:, 0], whole[:, 0]) and np.allclose(got[:, 1:], whole[:, 1:], rtol=1e-5, atol=1e-3)
both = [torch.zeros(12, device="cuda") for _ in range(world)]
dist.all_gather(both, torch.cat([bias, std]))
same = all(torch.equal(both[0], b) for b in both)
print(f"rank {rank}: global window sums match oracle: {ok}; coefficients identical on all ranks: {same}", flush=True)
dist.destroy_process_group()
sys.exit(0 if ok and same else 1)
