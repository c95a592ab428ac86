"""Child process of test_api_cpu.py: two gloo ranks train on halves of a batch
and must end with the tables one rank gets on the whole batch; then the
two-shard checkpoint is loaded into a single shard."""
import os
import sys

import torch
import torch.distributed as dist

import kraken_b200.pytorch as kk
from kraken_b200._native import C

out_dir = sys.argv[1]
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()

torch.manual_seed(0)
ids_all = torch.randint(0, 50, (8, 6))
g_all = torch.randn(3, 8, 6, 4)
gd_all = torch.randn(3, 8, 5)

kk.initialize("cpu", saved_dir=out_dir, seed=3)
kk.init_model("m", kk.OptimType.kAdagrad, {"initial_accumulator_value": "0.1"})
kk.update_lr(0.1)
ts = kk.register_sparse_table("e", 4, torch.float32, kk.InitializerType.kNormal, {})
td = kk.register_dense_table("w", torch.ones(5))
half = slice(rank * 4, rank * 4 + 4)
for s in range(3):
    kk.pull_sparse_table(ts, ids_all[half])
    kk.push_sparse_table(ts, ids_all[half], g_all[s, half])
    kk.push_dense_table(td, gd_all[s, half].sum(0))
rows = kk.pull_sparse_table(ts, torch.arange(50))
w = kk.pull_dense_table(td)
assert kk.try_save_model()

# single-shard oracle on the whole batch
shard = C.CpuShard(3)
shard.init_model("m", kk.OptimType.kAdagrad, {"initial_accumulator_value": "0.1"})
shard.create_sparse_table(0, "e", 4, kk.InitializerType.kNormal, {})
shard.create_dense_table(1, "w", torch.ones(5))
for s in range(3):
    uniq, inv = C.cpu_dedup(ids_all.reshape(-1))
    shard.pull_sparse(0, uniq)
    shard.push_sparse(0, uniq, C.cpu_segment_sum(g_all[s].reshape(-1, 4), inv, uniq.numel()), 0.1)
    shard.push_dense(1, gd_all[s].sum(0), 0.1)
want = shard.pull_sparse(0, torch.arange(50))
assert torch.allclose(rows, want, atol=1e-5), (rows - want).abs().max()
assert torch.allclose(w, shard.pull_dense(1), atol=1e-5)
if rank == 0:
    print("RANKS_MATCH_SINGLE ok")
kk.stop()
dist.barrier()

if rank == 0:
    from kraken_b200.checkpoint.manager import load_model
    from kraken_b200.runtime.cpu_engine import CpuEngine
    from kraken_b200.runtime.engine import EngineConfig

    eng = CpuEngine(EngineConfig(backend="cpu", seed=99), 0, 1)
    assert load_model(eng, out_dir)
    eng.update_lr(0.1)
    seen = torch.unique(ids_all)
    got = eng.pull_sparse_table(0, seen)
    assert torch.allclose(got, want[seen], atol=1e-6)
    assert eng.shard.sparse_size(0) == 50  # the final pull of arange(50) created every row
    assert torch.allclose(eng.pull_dense_table(1), w)
    print("RESHARD ok")
dist.barrier()
dist.destroy_process_group()
