"""Child process of test_gpu_multi.py: live reshard inside one job.  N ranks train two tables (Adam, so rows carry
two state slabs and a step count), halve the number of row-owning ranks, train on, go back to N owners, train on;
at every stage each row must sit on the rank the current owner function names, and at the end every row equals a
single CPU shard fed the same stream (scale-out / scale-in of kraken/ps/ps.cc:125-372, without a file)."""
import sys

import torch
import torch.distributed as dist

import kraken_b200.pytorch as kk
from kraken_b200._native import C
from kraken_b200.utils.hashing import owner_of

kk.initialize("gpu", seed=9, table_capacity=1 << 14, max_ids_per_call=20_000)
eng = kk.native.engine()
rank, world = eng.rank, eng.world
dev = torch.device("cuda", torch.cuda.current_device())
kk.init_model("m", kk.OptimType.kAdam, {})
kk.update_lr(0.02)
ta = kk.register_sparse_table("a", 8, torch.float32, kk.InitializerType.kConstant, {"value": "0.5"})
tb = kk.register_sparse_table("b", 4, torch.float32, kk.InitializerType.kConstant, {"value": "-0.25"})
shard = C.CpuShard(9)
shard.init_model("m", kk.OptimType.kAdam, {})
shard.create_sparse_table(ta, "a", 8, kk.InitializerType.kConstant, {"value": "0.5"})
shard.create_sparse_table(tb, "b", 4, kk.InitializerType.kConstant, {"value": "-0.25"})
gen = torch.Generator().manual_seed(0)
PER = 3000


def train(steps: int) -> None:
    for _ in range(steps):
        for t, dim in ((ta, 8), (tb, 4)):
            ids_all = torch.randint(0, 20_000, (world, PER), generator=gen)
            g_all = torch.randn(world, PER, dim, generator=gen)
            mine = ids_all[rank].to(dev)
            kk.pull_sparse_table(t, mine)
            kk.push_sparse_table(t, mine, g_all[rank].to(dev))
            uniq, inv = C.cpu_dedup(ids_all.reshape(-1))
            shard.pull_sparse(t, uniq)
            assert shard.push_sparse(t, uniq, C.cpu_segment_sum(g_all.reshape(-1, dim), inv, uniq.numel()), 0.02) == 0


def check_placement(owner_world: int) -> None:
    total = torch.zeros(2, dtype=torch.int64, device=dev)
    for k, t in enumerate((ta, tb)):
        ids = eng.sparse[t].export()["ids"].cpu()
        if ids.numel():
            assert bool((owner_of(0, ids, owner_world) == rank).all()), f"rank {rank} holds rows it does not own"
        assert rank < owner_world or ids.numel() == 0
        total[k] = ids.numel()
    dist.all_reduce(total)
    assert int(total[0]) == shard.sparse_size(ta) and int(total[1]) == shard.sparse_size(tb), total.tolist()


train(3)
check_placement(world)
moved_in = eng.reshard(max(1, world // 2))
check_placement(max(1, world // 2))
train(3)
moved_out = eng.reshard(world)
check_placement(world)
train(3)
eng.check()
probe = torch.arange(20_000)
for t in (ta, tb):
    got = kk.pull_sparse_table(t, probe.to(dev)).cpu()
    want = shard.pull_sparse(t, probe)
    assert torch.allclose(got, want, atol=2e-4), (t, float((got - want).abs().max()))
eng.check()
if rank == 0:
    print(f"LIVE_RESHARD ok world={world} rows_sent_by_rank0: {moved_in} in, {moved_out} out", flush=True)
kk.stop()
sys.exit(0)
