#!/usr/bin/env python
"""Pushes a fixed sequence of dense gradients through the UNMODIFIED reference's DCT emitter
(kraken/worker/dct_emitter.cc:16-43: error feedback, a top-k threshold refreshed every ``life_span`` pushes,
only entries at or above it travel) and writes the table values after every push to an .npz file.
Imports nothing from this repository's package."""
from __future__ import annotations

import argparse
import sys
import time

import numpy as np
import torch

STEPS, LIFE_SPAN, ETA, LR = 8, 3, 0.75, 0.1
BIG, SMALL = (30, 40), (10, 20)      # 1200 elements are compressed, 200 (< 256) travel dense


def inputs():
    g = torch.Generator().manual_seed(11)
    return [(torch.randn(*BIG, generator=g), torch.randn(*SMALL, generator=g)) for _ in range(STEPS)]


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref-path", required=True)
    ap.add_argument("--s-addr", required=True)
    ap.add_argument("--out", required=True)
    a = ap.parse_args()
    sys.path.insert(0, a.ref_path)
    import kraken.pytorch as kk  # the reference's package

    kk.initialize(a.s_addr, kk.EmitterType.kDCT, LIFE_SPAN, ETA)
    kk.init_model("dct", kk.OptimType.kSGD, {})
    kk.update_lr(LR)
    tb = kk.register_dense_table("big", torch.zeros(*BIG))
    ts = kk.register_dense_table("small", torch.zeros(*SMALL))
    out = {}
    for k, (gb, gs) in enumerate(inputs()):
        kk.push_dense_table(tb, gb)
        kk.push_dense_table(ts, gs)
        time.sleep(0.3)   # pushes are fire-and-forget in the reference
        out[f"big_{k}"] = kk.pull_dense_table(tb).numpy()
        out[f"small_{k}"] = kk.pull_dense_table(ts).numpy()
    np.savez(a.out, **out)
    kk.stop()
    return 0


if __name__ == "__main__":
    sys.exit(main())
