"""DeepFM on synthetic click data (counterpart of the reference's examples/DeepFM/main.py).

    python examples/deepfm/main.py                      # one process, GPU if present else CPU
    torchrun --nproc-per-node 8 examples/deepfm/main.py  # one rank per GPU
    python examples/deepfm/main.py --s_addr tcp://127.0.0.1:50000   # against scheduler_server + ps_server
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import kraken_b200.pytorch as kk  # noqa: E402
from kraken_b200.models import ClickDataset, DeepFM  # noqa: E402
from kraken_b200.ops import bce_with_logits  # noqa: E402


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--s_addr", default="auto")
    p.add_argument("--steps", type=int, default=200)
    p.add_argument("--batch", type=int, default=4096)
    p.add_argument("--fields", type=int, default=26)
    p.add_argument("--vocab", type=int, default=100_000)
    p.add_argument("--lr", type=float, default=1e-3)
    p.add_argument("--save_dir", default="")
    a = p.parse_args()

    kk.initialize(a.s_addr, saved_dir=a.save_dir)
    eng = kk.native.engine()
    dev = eng.device
    torch.manual_seed(0)
    model = DeepFM(a.fields, 13, 16, (400, 400, 400)).to(dev)
    opt = kk.Optimizer("deepfm", model.named_parameters(), a.lr, kk.Adam())
    data = ClickDataset(a.fields, 13, a.vocab, 1.1, seed=eng.rank)
    scale = 1.0 / eng.world
    for step in range(a.steps):
        dense, ids, labels = (t.to(dev) for t in data.batch(a.batch))
        loss = bce_with_logits(model(dense, ids), labels) * scale
        loss.backward()
        opt.step()
        if step % 20 == 0 and eng.rank == 0:
            print(f"step {step:4d}  loss {loss.item() * eng.world:.4f}")
    if a.save_dir:
        print("saved:", kk.try_save_model())
    kk.stop()


if __name__ == "__main__":
    main()
