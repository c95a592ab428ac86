#!/usr/bin/env python
"""Worker process of the reference on the CPU Wide&Deep configuration: 1 reference parameter server + 1
worker over localhost, fp32, batch 512, 200 steps, seed 0.  Drives ``kraken.pytorch`` as installed under
baseline/_ref (initialize, CombineEmbedding, Optimizer, Adagrad); imports nothing from this repository's package.

Model: 13 dense features (log1p of LogNormal(0, 1)), 26 single-hot fields with ids ~ Zipf(1.05) over 1e5 per
field, all fields hashed into one table per part - wide: dim-1 embeddings summed; deep: dim-8 embeddings
concatenated with the dense features, MLP 256-128-1 with ReLU; BCE-with-logits; server-side Adagrad lr 0.01
(the reference's Adagrad has no initial accumulator, kraken/ps/optim/adagrad.cc:18-48).  Labels from a fixed
random teacher.  Prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import sys
import time

import numpy as np
import torch

NUM_FIELDS, NUM_DENSE, VOCAB, DIM = 26, 13, 100_000, 8


def zipf_ids(rng, shape, vocab, s):
    u = rng.random(shape)
    a = 1.0 - s
    r = ((float(vocab + 1) ** a - 1.0) * u + 1.0) ** (1.0 / a) - 1.0
    return np.minimum(r.astype(np.int64), vocab - 1)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref-path", required=True)
    ap.add_argument("--s-addr", required=True)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--batch", type=int, default=512)
    ap.add_argument("--torch-threads", type=int, default=0)
    args = ap.parse_args()
    if args.torch_threads > 0:
        torch.set_num_threads(args.torch_threads)
    sys.path.insert(0, args.ref_path)
    import kraken.pytorch as kk  # the reference's package

    class WideAndDeep(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.emb = kk.CombineEmbedding([DIM, 1], initializers=[kk.NormalInitializer(0.0, 0.01),
                                                                    kk.ConstantInitializer(0.0)],
                                           names=["wd.deep", "wd.wide"])
            self.mlp = torch.nn.Sequential(torch.nn.Linear(NUM_FIELDS * DIM + NUM_DENSE, 256), torch.nn.ReLU(),
                                           torch.nn.Linear(256, 128), torch.nn.ReLU(), torch.nn.Linear(128, 1))

        def forward(self, dense, ids):
            e, w = self.emb([ids, ids])                # [B, F, 8], [B, F, 1]
            return w.sum(dim=(1, 2)) + self.mlp(torch.cat([e.flatten(1), dense], dim=1)).squeeze(-1)

    torch.manual_seed(0)
    rng = np.random.default_rng(0)
    t = np.random.default_rng(12345)
    w_dense, w_field = t.normal(0.0, 0.1, NUM_DENSE).astype(np.float32), t.normal(0.0, 0.1, NUM_FIELDS).astype(np.float32)
    base = (np.arange(NUM_FIELDS, dtype=np.int64) * VOCAB)[None, :]
    batches = []
    for _ in range(args.steps):
        dense = np.log1p(rng.lognormal(0.0, 1.0, (args.batch, NUM_DENSE))).astype(np.float32)
        ids = zipf_ids(rng, (args.batch, NUM_FIELDS), VOCAB, 1.05) + base
        h = ((ids * 2654435761) % (1 << 24)).astype(np.float32) / float(1 << 23) - 1.0
        logit = dense @ w_dense + h @ w_field
        labels = (rng.random(args.batch) < 1.0 / (1.0 + np.exp(-logit))).astype(np.float32)
        batches.append((torch.from_numpy(dense), torch.from_numpy(ids), torch.from_numpy(labels)))

    kk.initialize(args.s_addr)
    model = WideAndDeep()
    opt = kk.Optimizer("wide_deep", model.named_parameters(), 0.01, kk.Adagrad())
    loss_fn = torch.nn.BCEWithLogitsLoss()
    losses = []
    t0 = time.perf_counter()
    for dense, ids, labels in batches:
        loss = loss_fn(model(dense, ids), labels)
        loss.backward()
        opt.step()
        losses.append(float(loss.item()))
    dt = time.perf_counter() - t0
    print(json.dumps({"benchmark": "wide_deep_cpu", "impl": "reference", "engine": "1 ps_server + 1 worker, localhost ZeroMQ",
                      "steps": args.steps, "batch": args.batch, "samples_per_sec": args.steps * args.batch / dt,
                      "ms_per_step": dt / args.steps * 1e3, "loss_first10": sum(losses[:10]) / 10,
                      "loss_last10": sum(losses[-10:]) / 10, "torch_threads": torch.get_num_threads()}), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
