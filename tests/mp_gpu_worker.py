"""Child process of test_gpu_multi.py: N GPU ranks exchange rows and gradients through the
fused peer-memory kernels; the result must equal what one CPU shard computes on the
concatenated batch."""
import os
import sys

import torch
import torch.distributed as dist

import kraken_b200.pytorch as kk
from kraken_b200._native import C

out_dir = sys.argv[1]
EXCHANGE = sys.argv[2] if len(sys.argv) > 2 else "fused"
kk.initialize("gpu", seed=3, table_capacity=1 << 12, saved_dir=out_dir, exchange=EXCHANGE)
rank, world = dist.get_rank(), dist.get_world_size()
dev = torch.device("cuda", torch.cuda.current_device())
eng = kk.native.engine()

OPT, CONF, LR = kk.OptimType.kAdam, {"amsgrad": "true"}, 0.05
kk.init_model("m", OPT, CONF)
kk.update_lr(LR)
DIM, PER, STEPS = 8, 96, 4
ts = kk.register_sparse_table("e", DIM, torch.float32, kk.InitializerType.kNormal, {"stddev": "0.3"})
t1 = kk.register_sparse_table("e1", 1, torch.float32, kk.InitializerType.kConstant, {"value": "0.5"})
td = kk.register_dense_table("w", torch.linspace(-1, 1, 700).view(70, 10))
td2 = kk.register_dense_table("b", torch.ones(5))
# large enough that the fused dense step needs more blocks than fit on the GPU at once: its grid must
# stay resident (blocks wait for a flag raised after every block has finished), so it loops instead
BIG = (1200, 1024)
td3 = kk.register_dense_table("big", torch.full(BIG, 0.25))

torch.manual_seed(0)
ids_all = torch.randint(0, 200, (STEPS, world * PER))
g_all = torch.randn(STEPS, world * PER, DIM)
g1_all = torch.randn(STEPS, world * PER, 1)
gd_all = torch.randn(STEPS, world, 70, 10)
gd2_all = torch.randn(STEPS, world, 5)

shard = C.CpuShard(3)
shard.init_model("m", OPT, CONF)
shard.create_sparse_table(ts, "e", DIM, kk.InitializerType.kNormal, {"stddev": "0.3"})
shard.create_sparse_table(t1, "e1", 1, kk.InitializerType.kConstant, {"value": "0.5"})
shard.create_dense_table(td, "w", torch.linspace(-1, 1, 700).view(70, 10))
shard.create_dense_table(td2, "b", torch.ones(5))
shard.create_dense_table(td3, "big", torch.full(BIG, 0.25))

mine = slice(rank * PER, (rank + 1) * PER)
for s in range(STEPS):
    ids = ids_all[s, mine].to(dev)
    rows = kk.pull_sparse_table(ts, ids)
    rows1 = kk.pull_sparse_table(t1, ids)
    uniq, inv = C.cpu_dedup(ids_all[s])
    want = shard.pull_sparse(ts, uniq)[inv][mine]
    shard.pull_sparse(t1, uniq)
    assert torch.allclose(rows.cpu(), want, atol=1e-5), (s, (rows.cpu() - want).abs().max())
    kk.push_sparse_table(t1, ids, g1_all[s, mine].to(dev))
    kk.push_sparse_table(ts, ids, g_all[s, mine].to(dev))
    kk.push_dense_table(td, gd_all[s, rank].to(dev))
    kk.push_dense_table(td2, gd2_all[s, rank].to(dev))
    kk.push_dense_table(td3, torch.full(BIG, 0.01 * (rank + 1) * (s + 1), device=dev))
    w, b = kk.combine_pull_dense_table([td, td2])
    assert shard.push_sparse(ts, uniq, C.cpu_segment_sum(g_all[s], inv, uniq.numel()), LR) == 0
    assert shard.push_sparse(t1, uniq, C.cpu_segment_sum(g1_all[s], inv, uniq.numel()), LR) == 0
    shard.push_dense(td, gd_all[s].sum(0), LR)
    shard.push_dense(td2, gd2_all[s].sum(0), LR)
    shard.push_dense(td3, torch.full(BIG, 0.01 * (s + 1) * world * (world + 1) / 2), LR)
    assert torch.allclose(w.cpu(), shard.pull_dense(td).view(70, 10), atol=1e-5), s
    assert torch.allclose(b.cpu(), shard.pull_dense(td2), atol=1e-5), s
big = kk.pull_dense_table(td3).cpu()
assert torch.allclose(big, shard.pull_dense(td3).view(*BIG), atol=1e-5), (big - shard.pull_dense(td3).view(*BIG)).abs().max()
eng.check()
probe = torch.arange(200)
got = kk.pull_sparse_table(ts, probe.to(dev)).cpu()
shard_rows = shard.pull_sparse(ts, probe)
assert torch.allclose(got, shard_rows, atol=2e-4), (got - shard_rows).abs().max()
got1 = kk.pull_sparse_table(t1, probe.to(dev)).cpu()
assert torch.allclose(got1, shard.pull_sparse(t1, probe), atol=2e-4)
eng.check()
# every row lives on exactly one shard, the one OwnerOf names
local = eng.sparse[ts].export()["ids"].cpu().tolist()
assert all(C.owner_of(0, i, world) == rank for i in local)
cnt = torch.tensor([len(local)], device=dev)
dist.all_reduce(cnt)
assert int(cnt.item()) == 200
if rank == 0:
    print("MULTI_GPU_MATCHES_SINGLE ok")

if EXCHANGE != "fused":
    kk.stop()
    sys.exit(0)

# fused bag lookup across ranks
lens = torch.randint(0, 4, (40,), generator=torch.Generator().manual_seed(rank))
offsets = torch.cat([torch.zeros(1, dtype=torch.int64), lens.cumsum(0)])
values = torch.randint(0, 200, (int(offsets[-1]),), generator=torch.Generator().manual_seed(10 + rank))
pooled, ticket = eng.pull_sparse_pooled(ts, values.to(dev), offsets.to(dev), mean=True, patch_value=-1.0)
want = C.jagged_mean_forward(got[values], offsets, -1.0)
assert torch.allclose(pooled.cpu(), want, atol=1e-4)
eng.push_sparse_pooled(ts, ticket, torch.zeros(40, DIM, device=dev))
eng.check()
if rank == 0:
    print("MULTI_GPU_BAGS ok")

got = kk.pull_sparse_table(ts, probe.to(dev)).cpu()  # the zero-gradient Adam step above still moved rows
w_saved = w.cpu()  # parameter views die with the engine's arenas
assert kk.try_save_model()
kk.stop(keep_process_group=True)

# the same ranks load what they have just written into new engines: every rank reads its share of the shard
# files and routes the rows to their owners
kk.initialize("gpu", seed=17, table_capacity=1 << 10, exchange=EXCHANGE)
assert kk.try_load_model_blocked(out_dir)
eng2 = kk.native.engine()
ts2 = next(tid for tid, info in eng2.tables.items() if info.name == "e")
again = kk.pull_sparse_table(ts2, probe.to(dev)).cpu()
assert torch.allclose(again, got, atol=1e-6), "rows differ after the multi-rank load"
rows_now = torch.tensor([eng2.sparse[ts2].num_rows()], device=dev)
dist.all_reduce(rows_now)
assert int(rows_now.item()) == 200, f"{int(rows_now.item())} rows over all shards after the load"
eng2.check()
if rank == 0:
    print("MULTI_GPU_CHECKPOINT_LOAD ok")
kk.stop()

if rank == 0:
    from kraken_b200.checkpoint.manager import load_model
    from kraken_b200.runtime.cpu_engine import CpuEngine
    from kraken_b200.runtime.engine import EngineConfig

    cpu = CpuEngine(EngineConfig(backend="cpu", seed=99), 0, 1)
    assert load_model(cpu, out_dir)
    assert torch.allclose(cpu.pull_sparse_table(0, probe), got, atol=1e-6)
    assert cpu.shard.sparse_size(0) == 200
    assert torch.allclose(cpu.pull_dense_table(2), w_saved, atol=1e-6)
    assert torch.allclose(cpu.pull_dense_table(4), big, atol=1e-6)
    print("MULTI_GPU_CHECKPOINT_RESHARD ok")
