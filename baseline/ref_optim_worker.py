#!/usr/bin/env python
"""Runs one server-side optimizer of the UNMODIFIED reference (baseline/_ref) over a fixed sequence of pushes and
writes the table values after every push to an .npz file: the oracle of this framework's optimizer math
(kraken/ps/optim/{sgd,adagrad,adam,rmsprop}.cc).  Imports nothing from this repository's package.

A reference cluster holds ONE model (kraken/scheduler/scheduler.cc:154-190), so every optimizer configuration
needs a cluster of its own.  Rows start at a constant (the reference seeds its random initialisers from
std::random_device), gradients come from a seeded torch generator, the learning rate changes per step.
"""
from __future__ import annotations

import argparse
import json
import sys
import time

import numpy as np
import torch

STEPS, ROWS, DIM = 6, 40, 4


def inputs():
    g = torch.Generator().manual_seed(7)
    sparse = [torch.randn(ROWS, DIM, generator=g) for _ in range(STEPS)]
    dense = [torch.randn(3, 5, generator=g) for _ in range(STEPS)]
    # step 3 leaves some rows out (their state must not move) and repeats others (their gradients are summed first)
    ids = [torch.arange(ROWS, dtype=torch.int64) * 11 for _ in range(STEPS)]
    ids[3] = torch.cat([ids[3][:20], ids[3][:20]])
    lrs = [0.1, 0.05, 0.2, 0.1, 0.01, 0.3]
    return ids, sparse, dense, lrs


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref-path", required=True)
    ap.add_argument("--s-addr", required=True)
    ap.add_argument("--optim", required=True, help="Adagrad | Adam | RMSprop | SGD")
    ap.add_argument("--conf", default="{}", help="JSON object of string options")
    ap.add_argument("--out", required=True)
    a = ap.parse_args()
    sys.path.insert(0, a.ref_path)
    import kraken.pytorch as kk  # the reference's package

    kk.initialize(a.s_addr)
    kk.init_model("oracle", getattr(kk.OptimType, "k" + a.optim), json.loads(a.conf))
    ts = kk.register_sparse_table("e", DIM, torch.float32, kk.InitializerType.kConstant, {"value": "0.5"})
    td = kk.register_dense_table("w", torch.linspace(-1, 1, 15).view(3, 5))
    ids, sparse, dense, lrs = inputs()
    probe = torch.arange(ROWS, dtype=torch.int64) * 11
    kk.pull_sparse_table(ts, probe)
    out = {}
    for k in range(STEPS):
        kk.update_lr(lrs[k])
        kk.push_sparse_table(ts, ids[k], sparse[k])
        kk.push_dense_table(td, dense[k])
        time.sleep(0.3)   # pushes are fire-and-forget in the reference
        out[f"rows_{k}"] = kk.pull_sparse_table(ts, probe).numpy()
        out[f"dense_{k}"] = kk.pull_dense_table(td).numpy()
    np.savez(a.out, **out)
    kk.stop()
    return 0


if __name__ == "__main__":
    sys.exit(main())
