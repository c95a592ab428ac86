"""Wide & Deep with DCT gradient compression on the dense parameters (counterpart of the
reference's examples/WideAndDeep/main.py, which also selects EmitterType.kDCT).

    python examples/wide_deep/main.py [--multihot]
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import kraken_b200.pytorch as kk  # noqa: E402
from kraken_b200.models import ClickDataset, MultiHotDataset, MultiHotWideAndDeep, WideAndDeep  # noqa: E402
from kraken_b200.ops import bce_with_logits  # noqa: E402


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--s_addr", default="auto")
    p.add_argument("--steps", type=int, default=200)
    p.add_argument("--batch", type=int, default=512)
    p.add_argument("--multihot", action="store_true")
    a = p.parse_args()
    kk.initialize(a.s_addr, emitter_type=kk.EmitterType.kDCT, life_span=1000, eta=0.75)
    eng = kk.native.engine()
    dev = eng.device
    torch.manual_seed(0)
    if a.multihot:
        model = MultiHotWideAndDeep(20, 13, 16, (256, 128), mean_fields=range(0, 20, 2)).to(dev)
        data = MultiHotDataset(20, 13, 50_000, 1.1, mean_len=8, max_len=30, seed=eng.rank)
    else:
        model = WideAndDeep(26, 13, 8, (256, 128)).to(dev)
        data = ClickDataset(26, 13, 100_000, 1.05, seed=eng.rank)
    opt = kk.Optimizer("wide_deep", model.named_parameters(), 0.01, kk.Adagrad(initial_accumulator_value=0.1))
    for step in range(a.steps):
        batch = [t.to(dev) for t in data.batch(a.batch)]
        if a.multihot:
            dense, ids, offsets, labels = batch
            logits = model(dense, kk.JaggedTensor(ids, offsets, validate=False))
        else:
            dense, ids, labels = batch
            logits = model(dense, ids)
        loss = bce_with_logits(logits, labels) / eng.world
        loss.backward()
        opt.step()
        if step % 20 == 0 and eng.rank == 0:
            print(f"step {step:4d}  loss {loss.item() * eng.world:.4f}")
    kk.stop()


if __name__ == "__main__":
    main()
