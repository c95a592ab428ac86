"""Dense-only training: every parameter of an MLP is a dense table updated by the server-side
optimizer (counterpart of the reference's examples/Mnist/kraken/main.py, on synthetic images).

    python examples/mnist/main.py [--dct]
"""
import argparse
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import kraken_b200.pytorch as kk  # noqa: E402
from kraken_b200.models import MLP, mnist_like  # noqa: E402


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--s_addr", default="auto")
    p.add_argument("--steps", type=int, default=100)
    p.add_argument("--batch", type=int, default=64)
    p.add_argument("--dct", action="store_true")
    a = p.parse_args()
    kk.initialize(a.s_addr, emitter_type=kk.EmitterType.kDCT if a.dct else kk.EmitterType.kDefault)
    eng = kk.native.engine()
    dev = eng.device
    torch.manual_seed(0)
    model = MLP(784, [512, 256, 10]).to(dev)
    opt = kk.Optimizer("mnist", model.named_parameters(), 0.01, kk.SGD(momentum=0.9))
    rng = np.random.default_rng(eng.rank)
    means = np.random.default_rng(7).normal(0, 1, (10, 784)).astype(np.float32)
    for step in range(a.steps):
        x, y = (t.to(dev) for t in mnist_like(rng, means, a.batch))
        out = model(x)
        loss = torch.nn.functional.cross_entropy(out, y) / eng.world
        loss.backward()
        opt.step()
        if step % 10 == 0 and eng.rank == 0:
            acc = (out.argmax(1) == y).float().mean().item()
            print(f"step {step:4d}  loss {loss.item() * eng.world:.4f}  acc {acc:.3f}")
    kk.stop()


if __name__ == "__main__":
    main()
