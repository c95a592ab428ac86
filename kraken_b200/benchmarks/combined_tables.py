"""Pull + push of MANY small tables: one exchange per table against one exchange per row width.

The reference's DeepFM example keeps a dim-1 and a dim-4 table per field, 39 + 39 tables
(examples/DeepFM/model/DeepFM.py:64-69), and its combined calls send all of them in one request round per
server (kraken/worker/emitter.cc:185-278, :552-632).  This script times, on the same ids,

    per_table   pull_sparse_table / push_sparse_table once per table (78 exchanges),
    combined    combine_pull_sparse_table / combine_push_sparse_table (2 exchanges: widths 1 and 4),
    folded      ONE dim-8 table holding every field's row (ids offset per field; 1 exchange),

device-timed over ``--steps`` steps after ``--warmup``, max over ranks.

    torchrun --nproc-per-node N -m kraken_b200.benchmarks.combined_tables [--fields 39] [--batch 65536]
"""
import argparse

import torch

import kraken_b200.pytorch as kk
from kraken_b200.benchmarks.common import DeviceTimer, emit, world_rank
from kraken_b200.models.synthetic import zipf_ids
import numpy as np


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--fields", type=int, default=39)
    p.add_argument("--batch", type=int, default=65536, help="global batch: ids per table and step")
    p.add_argument("--vocab", type=int, default=1_000_000)
    p.add_argument("--steps", type=int, default=10)
    p.add_argument("--warmup", type=int, default=3)
    a = p.parse_args()
    world, rank = world_rank()
    B = a.batch // world
    F = a.fields
    kk.initialize("gpu", table_capacity=1 << 21, max_ids_per_call=0, seed=0)
    dev = torch.device("cuda", torch.cuda.current_device())
    eng = kk.native.engine()
    kk.init_model("m", kk.OptimType.kAdam, {})
    kk.update_lr(1e-3)
    dims = [1] * F + [4] * F
    tids = [kk.register_sparse_table(f"t{k}", d, torch.float32, kk.InitializerType.kNormal, {"stddev": "0.01"})
            for k, d in enumerate(dims)]
    folded = kk.register_sparse_table("folded", 8, torch.float32, kk.InitializerType.kNormal, {"stddev": "0.01"})
    rng = np.random.default_rng(3 + rank)
    total = a.warmup + a.steps
    per_field = [[torch.from_numpy(zipf_ids(rng, B, a.vocab, 1.1)).to(dev) for _ in range(F)] for _ in range(total)]
    grads = [torch.randn(B, d, device=dev) * 0.01 for d in dims]
    g_folded = torch.randn(B * F, 8, device=dev) * 0.01
    offs = (torch.arange(F, device=dev) * a.vocab).repeat_interleave(B)

    def per_table(s):
        ids = per_field[s] + per_field[s]
        rows = [kk.pull_sparse_table(t, i) for t, i in zip(tids, ids)]
        for t, i, g in zip(reversed(tids), reversed(ids), reversed(grads)):
            kk.push_sparse_table(t, i, g)
        return rows

    def combined(s):
        ids = per_field[s] + per_field[s]
        rows = kk.combine_pull_sparse_table(tids, ids)
        kk.combine_push_sparse_table(tids, ids, grads)
        return rows

    def one_table(s):
        ids = torch.cat(per_field[s]) + offs
        rows = kk.pull_sparse_table(folded, ids)
        kk.push_sparse_table(folded, ids, g_folded)
        return rows

    rec = {"benchmark": "combined_tables", "n_gpus": world, "tables": len(tids), "ids_per_table_per_gpu": B,
           "widths": "39 x dim 1 + 39 x dim 4" if F == 39 else f"{F} x dim 1 + {F} x dim 4"}
    timer = DeviceTimer()
    for name, fn in (("per_table", per_table), ("combined", combined), ("folded", one_table)):
        for s in range(a.warmup):
            fn(s)
        eng.check()
        l0 = eng.kernel_launches()
        timer.start()
        for s in range(a.warmup, total):
            fn(s)
        ms = timer.stop_ms()
        rec[f"{name}_us_per_step"] = round(ms / a.steps * 1e3, 1)
        rec[f"{name}_launches_per_step"] = (eng.kernel_launches() - l0) // a.steps
        eng.check()
    rec["combined_speedup_over_per_table"] = round(rec["per_table_us_per_step"] / rec["combined_us_per_step"], 2)
    rec["combined_over_folded"] = round(rec["combined_us_per_step"] / rec["folded_us_per_step"], 2)
    emit(rec)
    kk.stop()


if __name__ == "__main__":
    main()
