"""Child process of test_remote_cpu.py::test_several_workers_share_the_servers: one of several workers that push to
overlapping rows and dense tables of the same TCP deployment at the same time."""
import sys

import torch

import kraken_b200.pytorch as kk

s_addr, index, workers, steps = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), int(sys.argv[4])
kk.initialize(s_addr)
kk.init_model("shared", kk.OptimType.kSGD, {})            # idempotent: the first worker wins, the others attach
kk.update_lr(0.5)
ts = kk.register_sparse_table("e", 4, torch.float32, kk.InitializerType.kConstant, {"value": "0.0"})
td = kk.register_dense_table("w", torch.zeros(6, 5))
g = torch.Generator().manual_seed(100 + index)
for step in range(steps):
    ids = torch.randint(0, 300, (200,), generator=g)       # overlaps with every other worker's ids
    rows = kk.pull_sparse_table(ts, ids)
    assert rows.shape == (200, 4)
    kk.push_sparse_table(ts, ids, torch.full((200, 4), float(index + 1)))
    kk.push_dense_table(td, torch.full((6, 5), float(index + 1)))
    kk.pull_dense_table(td)
kk.stop()
print(f"TCP_WORKER {index} ok", flush=True)
