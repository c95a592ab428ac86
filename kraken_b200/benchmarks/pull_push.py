"""Huge-table stress: one dim-64 fp32 table with Adagrad state, ids ~ Zipf(0.9) over a large id
space, 26 single-hot fields, global batch 131072.  Measures the sparse pull and push alone (us per
step, device time, max over ranks) and the time to save / load the table in the checkpoint format.

    torchrun --nproc-per-node N -m kraken_b200.benchmarks.pull_push [--rows-per-gpu 20000000]
"""
import argparse
import tempfile
import time

import numpy as np
import torch

import kraken_b200.pytorch as kk
from kraken_b200.benchmarks.common import DeviceTimer, emit, sync_all, world_rank
from kraken_b200.models.synthetic import zipf_ids


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--global-batch", type=int, default=131072)
    p.add_argument("--rows-per-gpu", type=int, default=20_000_000, help="rows resident per shard before timing")
    p.add_argument("--id-space", type=int, default=1_000_000_000)
    p.add_argument("--checkpoint-rows", type=int, default=2_000_000, help="rows per shard in the save/load timing (0 = skip)")
    a = p.parse_args()
    world, rank = world_rank()
    n = a.global_batch // world * 26
    out_dir = tempfile.mkdtemp(prefix="kraken_ckpt_")
    kk.initialize("gpu", table_capacity=int(a.rows_per_gpu / 0.5), max_ids_per_call=max(n, 1 << 22), saved_dir=out_dir)
    dev = torch.device("cuda", torch.cuda.current_device())
    eng = kk.native.engine()
    kk.init_model("stress", kk.OptimType.kAdagrad, {"initial_accumulator_value": "0.1"})
    kk.update_lr(0.01)
    t = kk.register_sparse_table("big", 64, torch.float32, kk.InitializerType.kNormal, {"stddev": "0.01"})

    # populate: every rank pulls disjoint slices of the id space until its shard holds rows-per-gpu rows
    chunk = 1 << 22
    filled = 0
    base = rank * (a.id_space // world)
    while filled < a.rows_per_gpu * world // world:
        ids = torch.arange(base + filled, base + filled + chunk, device=dev)
        kk.pull_sparse_table(t, ids)
        filled += chunk
    sync_all()
    rows_local = eng.sparse[t].num_rows()

    rng = np.random.default_rng(5 + rank)
    total = a.warmup + a.steps
    batches = [torch.from_numpy(zipf_ids(rng, n, a.id_space, 0.9)).to(dev) for _ in range(total)]
    grads = torch.randn(n, 64, device=dev) * 0.01
    pull_t, push_t = DeviceTimer(), DeviceTimer()
    pull_ms = push_ms = 0.0
    for i in range(total):
        pull_t.start()
        rows = kk.pull_sparse_table(t, batches[i])
        ms_pull = pull_t.stop_ms()
        push_t.start()
        kk.push_sparse_table(t, batches[i], grads)
        ms_push = push_t.stop_ms()
        if i >= a.warmup:
            pull_ms += ms_pull
            push_ms += ms_push
    eng.check()
    rec = {"benchmark": "pull_push", "n_gpus": world, "global_batch": a.global_batch, "ids_per_gpu": n, "dim": 64,
           "rows_per_shard": rows_local, "pull_us": pull_ms / a.steps * 1e3, "push_us": push_ms / a.steps * 1e3}

    if a.checkpoint_rows > 0:
        # checkpoint timing on a shard trimmed to checkpoint-rows rows (the file format costs ~580 B per row)
        tab = eng.sparse[t]
        keep = tab.export()
        k = min(a.checkpoint_rows, int(keep["ids"].numel()))
        from kraken_b200._native import C
        C.table_clear(tab.host())
        tab.import_rows(keep["ids"][:k], keep["vals"][:k], {s: v[:k] for s, v in keep["states"].items()},
                        {s: v[:k] for s, v in keep["states_i"].items()})
        del keep
        sync_all()
        t0 = time.perf_counter()
        assert kk.try_save_model()
        sync_all()
        rec["save_s"] = time.perf_counter() - t0
        rec["checkpoint_rows_per_shard"] = k
        kk.stop()
        kk.initialize("gpu", table_capacity=int(k / 0.5))
        t0 = time.perf_counter()
        assert kk.try_load_model_blocked(out_dir)
        sync_all()
        rec["load_s"] = time.perf_counter() - t0
    emit(rec)
    kk.stop()


if __name__ == "__main__":
    main()
