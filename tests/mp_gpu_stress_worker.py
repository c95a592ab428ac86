"""Child process of test_gpu_multi.py: back-to-back sparse exchanges with nothing in between.

Every rank pulls and pushes two tables for many steps without a dense step, a host
synchronisation or any other collective between them, first launched eagerly and then as replays
of one captured CUDA graph, with ``overlap_dense_step=True`` as the benchmark runs.  The id stream
is Zipf-skewed and arranged so that rank 0 owns about half of all rows: ranks therefore finish
their phases at visibly different times, which is when a rank that runs ahead could disturb a
slower owner (overwritten inbox words, a push applied twice or not at all).  At the end every row
(Adam: a lost or doubled update moves a value by about lr) must equal what one CPU shard computes on the concatenated
stream - the scenario of the reference's emitter test (kraken/test/worker/emitter_test.cc:89-158)
at scale.
"""
import sys
import time

import numpy as np
import torch
import torch.distributed as dist

import kraken_b200.pytorch as kk
from kraken_b200._native import C
from kraken_b200.utils.hashing import owner_of

PER = int(sys.argv[1]) if len(sys.argv) > 1 else 200_000      # ids per rank, table and step
STEPS = int(sys.argv[2]) if len(sys.argv) > 2 else 50
POOL = 1_500_000
DIM_A, DIM_B = 8, 4
LR = 0.01

kk.initialize("gpu", seed=5, table_capacity=1 << 22, max_ids_per_call=PER, overlap_dense_step=True)
eng = kk.native.engine()
rank, world = eng.rank, eng.world
dev = torch.device("cuda", torch.cuda.current_device())


def barrier():
    if world > 1:
        dist.barrier()


def broadcast(t):
    if world > 1:
        dist.broadcast(t, 0)


def all_reduce(t, op=dist.ReduceOp.SUM):
    if world > 1:
        dist.all_reduce(t, op=op)


kk.init_model("stress", kk.OptimType.kAdam, {})
kk.update_lr(LR)
ta = kk.register_sparse_table("a", DIM_A, torch.float32, kk.InitializerType.kConstant, {"value": "0.25"})
tb = kk.register_sparse_table("b", DIM_B, torch.float32, kk.InitializerType.kConstant, {"value": "-0.5"})

# id pool: half of it owned by rank 0, the rest spread over the other ranks
g = torch.Generator().manual_seed(1234)
cand = torch.randint(0, 1 << 40, (POOL * 4,), generator=g)
own = owner_of(0, cand, world)
zero, rest = cand[own == 0], cand[own != 0] if world > 1 else cand[:0]
half = POOL // 2 if world > 1 else POOL
pool = torch.cat([zero[:half], rest[:POOL - half]])
pool = pool[torch.randperm(pool.numel(), generator=g)]


def zipf_index(gen: np.random.Generator, n: int) -> np.ndarray:
    u = gen.random(n)
    a = 1.0 - 1.05
    r = ((float(pool.numel() + 1) ** a - 1.0) * u + 1.0) ** (1.0 / a) - 1.0
    return np.minimum(r.astype(np.int64), pool.numel() - 1)


def ids_of(step: int, r: int, table: int) -> torch.Tensor:
    gen = np.random.default_rng(100_000 * table + 1000 * step + r)
    return pool[torch.from_numpy(zipf_index(gen, PER))]


def grad_of(ids: torch.Tensor, step: int, dim: int) -> torch.Tensor:
    """Exact on every device: small integers scaled by a power of two."""
    d = torch.arange(dim, device=ids.device, dtype=torch.int64)
    v = ((ids.unsqueeze(1) % 1000003) * 8191 + d * 97 + step * 131) % 1024
    return (v.to(torch.float32) - 512.0) / 4096.0


ids_a = torch.stack([ids_of(s, rank, 0) for s in range(STEPS)]).to(dev)
ids_b = torch.stack([ids_of(s, rank, 1) for s in range(STEPS)]).to(dev)


def one_step(ia: torch.Tensor, ib: torch.Tensor, ga: torch.Tensor, gb: torch.Tensor) -> None:
    kk.pull_sparse_table(ta, ia)
    kk.pull_sparse_table(tb, ib)
    kk.push_sparse_table(tb, ib, gb)   # reverse order, as autograd would push
    kk.push_sparse_table(ta, ia, ga)


torch.cuda.synchronize()
barrier()
t0 = time.perf_counter()
eager_steps = STEPS // 2
for s in range(eager_steps):
    one_step(ids_a[s], ids_b[s], grad_of(ids_a[s], s, DIM_A), grad_of(ids_b[s], s, DIM_B))

# the second half: one captured step, replayed with new ids copied into its input buffers
buf_a, buf_b = ids_a[eager_steps].clone(), ids_b[eager_steps].clone()
step_no = torch.zeros(1, dtype=torch.int64, device=dev)


def graph_body() -> None:
    d_a = torch.arange(DIM_A, device=dev, dtype=torch.int64)
    d_b = torch.arange(DIM_B, device=dev, dtype=torch.int64)
    ga = ((((buf_a.unsqueeze(1) % 1000003) * 8191 + d_a * 97 + step_no * 131) % 1024).to(torch.float32) - 512.0) / 4096.0
    gb = ((((buf_b.unsqueeze(1) % 1000003) * 8191 + d_b * 97 + step_no * 131) % 1024).to(torch.float32) - 512.0) / 4096.0
    one_step(buf_a, buf_b, ga, gb)


torch.cuda.synchronize()
side = torch.cuda.Stream()
graph = torch.cuda.CUDAGraph()
step_no.fill_(eager_steps)
with torch.cuda.stream(side):
    with torch.cuda.graph(graph, stream=side):
        graph_body()
# capture executes nothing: the captured step has not run yet
for s in range(eager_steps, STEPS):
    buf_a.copy_(ids_a[s])
    buf_b.copy_(ids_b[s])
    step_no.fill_(s)
    graph.replay()
torch.cuda.synchronize()
elapsed = time.perf_counter() - t0
eng.check()
barrier()

# ------------------------------------------------------------------ oracle on rank 0, compare everywhere
exp_a, exp_b = eng.sparse[ta].export(), eng.sparse[tb].export()
ok = torch.ones(1, device=dev)
if rank == 0:
    shard = C.CpuShard(5)
    shard.init_model("stress", kk.OptimType.kAdam, {})
    shard.create_sparse_table(ta, "a", DIM_A, kk.InitializerType.kConstant, {"value": "0.25"})
    shard.create_sparse_table(tb, "b", DIM_B, kk.InitializerType.kConstant, {"value": "-0.5"})
    for s in range(STEPS):
        for t, dim, tab in ((ta, DIM_A, 0), (tb, DIM_B, 1)):
            all_ids = torch.cat([ids_of(s, r, tab) for r in range(world)])
            uniq, inv = C.cpu_dedup(all_ids)
            shard.pull_sparse(t, uniq)
            assert shard.push_sparse(t, uniq, C.cpu_segment_sum(grad_of(all_ids, s, dim), inv, uniq.numel()), LR) == 0
else:
    shard = None

# every rank checks its own rows against rank 0's oracle: rank 0 broadcasts (ids, values, steps) per table
for t, exp, dim in ((ta, exp_a, DIM_A), (tb, exp_b, DIM_B)):
    if rank == 0:
        seen = torch.unique(torch.cat([ids_of(s, r, 0 if t == ta else 1) for s in range(STEPS) for r in range(world)]))
        want = shard.pull_sparse(t, seen)
        meta = torch.tensor([seen.numel()], device=dev)
    else:
        meta = torch.zeros(1, dtype=torch.int64, device=dev)
    broadcast(meta)
    n = int(meta.item())
    all_ids = seen.to(dev) if rank == 0 else torch.empty(n, dtype=torch.int64, device=dev)
    all_val = want.to(dev) if rank == 0 else torch.empty((n, dim), dtype=torch.float32, device=dev)
    broadcast(all_ids)
    broadcast(all_val)
    mine = owner_of(0, all_ids, world).to(dev) == rank
    rows, found = eng.sparse[t].lookup(all_ids[mine])
    total = torch.tensor([int(exp["ids"].numel())], device=dev)
    all_reduce(total)
    bad = []
    if not bool(found.all()):
        bad.append(f"{int((~found.bool()).sum())} rows missing")
    err = (rows - all_val[mine]).abs().max().item() if rows.numel() else 0.0
    if err > 2e-3:
        bad.append(f"max value error {err:.4g}")
    if int(total.item()) != n:
        bad.append(f"{int(total.item())} rows over all shards, expected {n}")
    if bad:
        print(f"rank {rank} table {t}: " + "; ".join(bad), flush=True)
        ok.zero_()
# a call longer than the exchange buffers, of a different length on every rank: the ranks agree on the
# number of rounds and the shorter ones join the later rounds with no ids
tc = kk.register_sparse_table("c", 4, torch.float32, kk.InitializerType.kConstant, {"value": "0.5"})
eng.cfg.long_id_streams = True
n_long = (rank + 1) * PER + PER // 3 + 17
long_ids = torch.arange(n_long, device=dev) * 13 + (1 << 41)      # ranks overlap: rank r's ids contain rank r-1's
for _ in range(2):
    got = kk.pull_sparse_table(tc, long_ids)
    if got.shape != (n_long, 4) or not bool((got == 0.5).all()):
        print(f"rank {rank}: long id stream came back wrong", flush=True)
        ok.zero_()
    kk.push_sparse_table(tc, long_ids, torch.zeros(n_long, 4, device=dev))   # Adam with zero gradients moves nothing
rows_c = torch.tensor([eng.sparse[tc].num_rows()], device=dev)
all_reduce(rows_c)
if int(rows_c.item()) != world * PER + PER // 3 + 17:
    print(f"rank {rank}: table c holds {int(rows_c.item())} rows over all shards", flush=True)
    ok.zero_()
eng.cfg.long_id_streams = False

all_reduce(ok, dist.ReduceOp.MIN)
eng.check()
if rank == 0:
    rows_a = int(exp_a["ids"].numel())
    print(f"STRESS world={world} ids/rank/table={PER} steps={STEPS} ({eager_steps} eager + {STEPS - eager_steps} graph replays) "
          f"rank0_rows_a={rows_a} wall={elapsed:.2f}s", flush=True)
    print("MULTI_GPU_STRESS ok" if ok.item() == 1 else "MULTI_GPU_STRESS FAILED", flush=True)
kk.stop()
sys.exit(0 if ok.item() == 1 else 1)
