"""Huge-table stress: one dim-64 fp32 table with Adagrad state, ids ~ Zipf(0.9) over a large id
space, 26 single-hot fields, global batch 131072.  Measures the sparse pull and push alone (us per
step, device time, max over ranks) and the time to save / load the table in the checkpoint format.

    torchrun --nproc-per-node N -m kraken_b200.benchmarks.pull_push [--rows-per-gpu 20000000]
"""
import argparse
import os
import tempfile
import time

import numpy as np
import torch

import kraken_b200.pytorch as kk
from kraken_b200.benchmarks.common import (DeviceTimer, NvlinkCounters, emit, measure_copy_gbs, measure_peer_gbs, sync_all,
                                            world_rank)
from kraken_b200.models.synthetic import zipf_ids


def roofline(ex: dict, dim: int, pull_us: float, push_us: float, created: float, hbm_gbs: float, link_gbs: float) -> dict:
    """Lower bounds of one rank's pull and push from the bytes they must move: over NVLink (per direction,
    at ``link_gbs``) and through HBM (algorithmic bytes at ``hbm_gbs``) - both rates measured by this run
    unless given on the command line; the bound is the slower of the two and the fraction is bound / measured time."""
    n, u, row = ex["occurrences"], ex["unique"], dim * 4
    # pull: read ids, write + read the occurrence map, gather owned rows (about u rows per rank: read + write),
    # read the received rows once and write the expanded [n, dim] result
    # (+ value and accumulator rows written for every row the pull creates)
    pull_hbm = n * 8 + 2 * n * 4 + 2 * u * row + u * row + n * row + 2 * created * row
    # push: read [n, dim] gradients, red-add into u rows (read-modify-write), copy them to the inbox
    # (read + write), then read them and read-modify-write value and accumulator rows
    push_hbm = n * row + 2 * u * row + 2 * u * row + u * row + 4 * u * row
    pull_link = max(ex["pull_bytes_in"], ex["pull_bytes_out"])
    push_link = ex["push_bytes_out"]
    out = {"unique_per_gpu": u, "unique_remote_per_gpu": ex["unique_remote"], "hbm_copy_gbs": round(hbm_gbs, 1),
           "peer_copy_gbs_per_direction": round(link_gbs, 1)}
    for name, hbm, link, t in (("pull", pull_hbm, pull_link, pull_us), ("push", push_hbm, push_link, push_us)):
        hbm_us, link_us = hbm / (hbm_gbs * 1e3), (link / (link_gbs * 1e3) if link_gbs > 0 else 0.0)
        bound = max(hbm_us, link_us)
        out[f"{name}_hbm_bound_us"] = round(hbm_us, 1)
        out[f"{name}_nvlink_bound_us"] = round(link_us, 1)
        out[f"{name}_roofline_fraction"] = round(bound / t, 3) if t > 0 else None
    return out


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--global-batch", type=int, default=131072)
    p.add_argument("--rows-per-gpu", type=int, default=20_000_000, help="rows resident per shard before timing")
    p.add_argument("--id-space", type=int, default=1_000_000_000)
    p.add_argument("--resident-ids", action="store_true",
                   help="draw the ids from the rows populated before timing (steady state: no row is created in the "
                        "timed steps) instead of from the whole id space (nearly every unique id is a new row)")
    p.add_argument("--graph", action="store_true",
                   help="replay the pull and the push as two CUDA graphs (as inside a captured training step) "
                        "instead of launching their kernels from Python")
    p.add_argument("--checkpoint-rows", type=int, default=2_000_000, help="rows per shard in the save/load timing (0 = skip)")
    p.add_argument("--hbm-gbs", type=float, default=0.0, help="copy bandwidth for the roofline (0 = measure it here)")
    p.add_argument("--link-gbs", type=float, default=0.0,
                   help="peer-copy bandwidth per direction for the roofline (0 = measure it here with rank -> rank + 1 copies)")
    a = p.parse_args()
    world, rank = world_rank()
    n = a.global_batch // world * 26
    # one directory for all ranks: they share the launcher as parent process
    out_dir = os.path.join(tempfile.gettempdir(), f"kraken_ckpt_{os.getppid()}_{os.environ.get('MASTER_PORT', '0')}")
    os.makedirs(out_dir, exist_ok=True)
    # room for the resident rows plus the rows the timed steps create (ids are drawn from a wide space, so
    # most of every batch is new), at a load factor of 0.6
    capacity = int((a.rows_per_gpu + (a.warmup + a.steps) * n * 0.8) / 0.6)
    kk.initialize("gpu", table_capacity=capacity, max_ids_per_call=max(n, 1 << 22), saved_dir=out_dir)
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
    if a.resident_ids:
        # rank r populated [r * S, r * S + filled): spread Zipf ranks over those slices
        S = a.id_space // world
        batches = []
        for _ in range(total):
            k = torch.from_numpy(zipf_ids(rng, n, world * filled, 0.9))
            batches.append(((k % world) * S + k // world).to(dev))
    else:
        batches = [torch.from_numpy(zipf_ids(rng, n, a.id_space, 0.9)).to(dev) for _ in range(total)]
    rows_before = None
    grads = torch.randn(n, 64, device=dev) * 0.01
    pull_t, push_t = DeviceTimer(), DeviceTimer()
    pull_ms = push_ms = 0.0
    g_pull = g_push = None
    if a.graph:
        static_ids = batches[0].clone()
        for _ in range(2):  # eager: creates the channel and fills the allocator pool
            kk.pull_sparse_table(t, static_ids)
            kk.push_sparse_table(t, static_ids, grads)
        sync_all()
        g_pull, g_push = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
        with torch.cuda.graph(g_pull):
            rows = kk.pull_sparse_table(t, static_ids)
        with torch.cuda.graph(g_push, pool=g_pull.pool()):
            kk.push_sparse_table(t, static_ids, grads)
        sync_all()
    for i in range(total):
        if g_pull is not None:
            static_ids.copy_(batches[i])
            pull_t.start()
            g_pull.replay()
            ms_pull = pull_t.stop_ms()
            push_t.start()
            g_push.replay()
            ms_push = push_t.stop_ms()
        else:
            pull_t.start()
            rows = kk.pull_sparse_table(t, batches[i])
            ms_pull = pull_t.stop_ms()
            push_t.start()
            kk.push_sparse_table(t, batches[i], grads)
            ms_push = push_t.stop_ms()
        if i >= a.warmup:
            pull_ms += ms_pull
            push_ms += ms_push
        elif i == a.warmup - 1:
            rows_before = eng.sparse[t].num_rows()
    eng.check()
    created = (eng.sparse[t].num_rows() - (rows_before or rows_local)) / max(1, a.steps)
    rec = {"benchmark": "pull_push", "n_gpus": world, "global_batch": a.global_batch, "ids_per_gpu": n, "dim": 64,
           "rows_per_shard": rows_local, "pull_us": pull_ms / a.steps * 1e3, "push_us": push_ms / a.steps * 1e3}
    rec["ids"] = "resident rows" if a.resident_ids else "whole id space"
    rec["launch"] = "cuda-graph replay" if a.graph else "eager"
    rec["rows_created_per_step"] = round(created)
    hbm_gbs = a.hbm_gbs or measure_copy_gbs(dev)
    link_gbs = a.link_gbs or measure_peer_gbs()
    ex = eng.metrics()["big"]["last_exchange"]
    rec.update(roofline(ex, 64, rec["pull_us"], rec["push_us"], created, hbm_gbs, link_gbs))

    if world > 1 and g_pull is not None:
        # measured link traffic of the fused kernels: NVML's NVLink byte counters around 50 replays of the pull
        # alone and 50 of the push alone (same ids), next to the bytes the exchange counts predict
        nvl = NvlinkCounters(dev)
        reps = 50

        def traffic(graph):
            sync_all()
            time.sleep(0.2)          # the counters are sampled by the driver, not updated per packet
            a = nvl.read()
            for _ in range(reps):
                graph.replay()
            sync_all()
            time.sleep(0.2)
            b = nvl.read()
            return None if a is None or b is None else ((b[0] - a[0]) / reps, (b[1] - a[1]) / reps)

        t_pull, t_push = traffic(g_pull), traffic(g_push)
        if t_pull is None or t_push is None:
            rec["nvlink_counters"] = "not exposed by the driver here: " + nvl.why
        else:
            rec["nvlink_counters"] = {
                "pull_tx_bytes": round(t_pull[0]), "pull_rx_bytes": round(t_pull[1]),
                "pull_expected_out": ex["pull_bytes_out"], "pull_expected_in": ex["pull_bytes_in"],
                "push_tx_bytes": round(t_push[0]), "push_rx_bytes": round(t_push[1]),
                "push_expected_out": ex["push_bytes_out"],
                "note": "per launch sequence and GPU; expected = remote unique rows x row bytes (+ 8 B per id sent); "
                        "rx of a push and tx of a pull are the other ranks' rows for this shard, about the same size"}

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
        kk.stop(keep_process_group=True)
        kk.initialize("gpu", table_capacity=int(k / 0.5))
        t0 = time.perf_counter()
        assert kk.try_load_model_blocked(out_dir)
        sync_all()
        rec["load_s"] = time.perf_counter() - t0
        eng2 = kk.native.engine()
        rec["rows_after_load_per_shard"] = int(next(iter(eng2.sparse.values())).num_rows())
        rec["checkpoint_gb_per_shard"] = round(os.path.getsize(max(
            (os.path.join(dp, f) for dp, _, fs in os.walk(out_dir) for f in fs if f.endswith(".sparse")),
            key=os.path.getsize)) / 1e9, 2)
    emit(rec)
    kk.stop()


if __name__ == "__main__":
    main()
