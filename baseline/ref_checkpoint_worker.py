#!/usr/bin/env python
"""Worker of the checkpoint cross-check, run against the UNMODIFIED reference (baseline/_ref): either trains a
small model and has the reference write a checkpoint (``--mode save``), or has the reference load a checkpoint
directory - written by anyone - and reports what it serves afterwards (``--mode load``).  Imports nothing from
this repository's package.  The numbers the test compares go to an .npz file.

Model: Adam with amsgrad (the richest per-row state: first and second moment, their maximum, a step counter),
one sparse table "e" of width 4, one dense table "w" of shape [5, 3].
"""
from __future__ import annotations

import argparse
import sys
import time

import numpy as np
import torch

LR = 0.05


def ids_of() -> torch.Tensor:
    small = torch.arange(0, 300, dtype=torch.int64) * 7919
    big = (1 << 40) + torch.arange(0, 50, dtype=torch.int64) * 104729
    return torch.cat([small, big])


def grads(seed: int, n: int):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(n, 4, generator=g), torch.randn(5, 3, generator=g)


def settle():
    """The reference's pushes are fire-and-forget (kraken/worker/emitter.cc:431-446): give them time to land."""
    time.sleep(0.5)


def wait_until_written(saved_dir: str, shards: int, timeout_s: float = 60.0) -> bool:
    """The reference answers TrySaveModel when its servers have QUEUED the save (kraken/ps/ps.cc:487-520); a push
    sent right behind it can land in some rows before they are written.  Returns once every shard directory holds
    router, model and table files whose sizes have stopped changing."""
    import os

    def snapshot():
        dirs = sorted(d for d in os.listdir(saved_dir) if d.startswith("shard_"))
        if len(dirs) < shards:
            return None
        sizes = {}
        for d in dirs:
            stamps = sorted(os.listdir(os.path.join(saved_dir, d)))
            if not stamps:
                return None
            last = os.path.join(saved_dir, d, stamps[-1])
            names = os.listdir(last)
            if not all(f in names for f in ("model.binary", "router.binary", "e.sparse")):
                return None
            for f in names:
                sizes[os.path.join(last, f)] = os.path.getsize(os.path.join(last, f))
        return sizes

    t0, before = time.time(), None
    while time.time() - t0 < timeout_s:
        now = snapshot()
        if now is not None and now == before:
            return True
        before = now
        time.sleep(0.3)
    return False


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref-path", required=True)
    ap.add_argument("--s-addr", required=True)
    ap.add_argument("--mode", choices=("save", "load"), required=True)
    ap.add_argument("--dir", default="", help="checkpoint directory to load (mode load)")
    ap.add_argument("--out", required=True, help=".npz file for the numbers")
    ap.add_argument("--saved-dir", default="", help="mode save: the servers' --saved_dir, watched until the files are complete")
    ap.add_argument("--shards", type=int, default=1, help="mode save: how many servers write")
    a = ap.parse_args()
    sys.path.insert(0, a.ref_path)
    import kraken.pytorch as kk  # the reference's package

    kk.initialize(a.s_addr)
    ids = ids_of()
    g1, d1 = grads(1, ids.numel())
    g2, d2 = grads(2, ids.numel())
    out = {}
    if a.mode == "save":
        kk.init_model("ckpt", kk.OptimType.kAdam, {"amsgrad": "true"})
        kk.update_lr(LR)
        ts = kk.register_sparse_table("e", 4, torch.float32, kk.InitializerType.kNormal, {"mean": "0.0", "stddev": "0.1"})
        td = kk.register_dense_table("w", torch.linspace(-1, 1, 15).view(5, 3))
        kk.pull_sparse_table(ts, ids)
        kk.push_sparse_table(ts, ids, g1)
        kk.push_dense_table(td, d1)
        settle()
        out["rows_at_save"] = kk.pull_sparse_table(ts, ids).numpy()
        out["dense_at_save"] = kk.pull_dense_table(td).numpy()
        if not kk.try_save_model():
            print("the reference refused to save", file=sys.stderr)
            return 2
        if a.saved_dir and not wait_until_written(a.saved_dir, a.shards):
            print("the checkpoint files did not appear under " + a.saved_dir, file=sys.stderr)
            return 2
    else:
        if not kk.try_load_model_blocked(a.dir):
            print("the reference could not load " + a.dir, file=sys.stderr)
            return 2
        kk.update_lr(LR)
        # tables are found again by name (the scheduler's registry deduplicates, kraken/scheduler/scheduler.cc:192-321)
        ts = kk.register_sparse_table("e", 4, torch.float32, kk.InitializerType.kNormal, {"mean": "0.0", "stddev": "0.1"})
        td = kk.register_dense_table("w", torch.linspace(-1, 1, 15).view(5, 3))
        out["rows_at_save"] = kk.pull_sparse_table(ts, ids).numpy()
        out["dense_at_save"] = kk.pull_dense_table(td).numpy()
    # one more update from the saved state: only right if the optimizer state and step counters came along
    kk.push_sparse_table(ts, ids, g2)
    kk.push_dense_table(td, d2)
    settle()
    out["rows_after"] = kk.pull_sparse_table(ts, ids).numpy()
    out["dense_after"] = kk.pull_dense_table(td).numpy()
    out["table_ids"] = np.array([ts, td])
    np.savez(a.out, **out)
    kk.stop()
    return 0


if __name__ == "__main__":
    sys.exit(main())
