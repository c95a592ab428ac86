#!/usr/bin/env python
"""One training script, two packages: with ``--impl reference`` the name ``kraken.pytorch`` is the UNMODIFIED
reference (baseline/_ref, talking to its own scheduler and server processes); with ``--impl ours`` it is this
framework behind ``kraken_b200.install_alias()``.  Everything after the import is the same code, written against
the reference's public API (kraken/pytorch/__init__.py:3-35): Embedding, CombineEmbedding, Optimizer, Adam.
Writes the loss of every step and the final dense parameters to an .npz file.

Model: Wide&Deep on 6 fields - wide dim-1 and deep dim-4 embeddings (one CombineEmbedding), 3 dense features,
MLP 16-8-1.  Rows start at a constant (the reference seeds its random initialisers from std::random_device);
the dense layers are initialised by torch under a fixed seed, which both runs share.
"""
from __future__ import annotations

import argparse
import sys
import time

import numpy as np
import torch

FIELDS, DENSE, STEPS, BATCH, VOCAB = 6, 3, 25, 64, 50


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", choices=("reference", "ours"), required=True)
    ap.add_argument("--ref-path", default="")
    ap.add_argument("--s-addr", required=True, help="scheduler address of the reference cluster, or cpu / gpu for ours")
    ap.add_argument("--out", required=True)
    a = ap.parse_args()
    if a.impl == "reference":
        sys.path.insert(0, a.ref_path)
    else:
        import kraken_b200
        kraken_b200.install_alias()
    import kraken.pytorch as kk

    class WideAndDeep(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.emb = kk.CombineEmbedding([4, 1], initializers=[kk.ConstantInitializer(0.05), kk.ConstantInitializer(0.0)],
                                           names=["deep", "wide"])
            self.mlp = torch.nn.Sequential(torch.nn.Linear(FIELDS * 4 + DENSE, 16), torch.nn.ReLU(),
                                           torch.nn.Linear(16, 8), torch.nn.ReLU(), torch.nn.Linear(8, 1))

        def forward(self, dense, ids):
            e, w = self.emb([ids, ids])
            return w.sum(dim=(1, 2)) + self.mlp(torch.cat([e.flatten(1), dense], dim=1)).squeeze(-1)

    torch.manual_seed(0)
    g = torch.Generator().manual_seed(1)
    batches = []
    for _ in range(STEPS):
        ids = torch.randint(0, VOCAB, (BATCH, FIELDS), generator=g) + torch.arange(FIELDS) * VOCAB
        dense = torch.randn(BATCH, DENSE, generator=g)
        labels = (torch.rand(BATCH, generator=g) < torch.sigmoid(dense.sum(1) + (ids[:, 0] % 3 - 1).float())).float()
        batches.append((dense, ids, labels))

    kk.initialize(a.s_addr)
    model = WideAndDeep()
    opt = kk.Optimizer("dropin", model.named_parameters(), 0.02, kk.Adam())
    loss_fn = torch.nn.BCEWithLogitsLoss()
    losses = []
    for dense, ids, labels in batches:
        loss = loss_fn(model(dense, ids), labels)
        loss.backward()
        if a.impl == "reference":
            time.sleep(0.15)      # its pushes are fire-and-forget: let them land before the parameters are pulled
        opt.step()
        losses.append(float(loss.item()))
    out = {"losses": np.array(losses)}
    for k, p in enumerate(model.mlp.parameters()):
        out[f"param_{k}"] = p.detach().numpy().copy()
    np.savez(a.out, **out)
    kk.stop()
    return 0


if __name__ == "__main__":
    sys.exit(main())
