#!/usr/bin/env python
"""Worker process of the reference arm: trains the benchmark's DeepFM configuration through the
reference's own public API (``kraken.pytorch`` as installed under baseline/_ref: initialize,
CombineEmbedding, Optimizer, Adam), the way examples/DeepFM/main.py:15-35 of the reference drives
its example.  Runs on the CPU in fp32, as everything in the reference does.  Imports nothing from
this repository's package, so none of its native libraries are loaded.

Model (the DeepFM configuration of the benchmark): 26 single-hot fields over 1e7 ids each, one
dim-16 table for the second-order / deep embeddings and one dim-1 table for the first-order
weights (both pulled in ONE request round through CombineEmbedding, the reference's cheapest
path), FM second-order term, MLP 400-400-400-1 with ReLU, BCE-with-logits, server-side Adam lr 1e-3.
Synthetic data: the same generator as the benchmark's own arm (log1p-LogNormal dense features,
Zipf(1.1) ids, labels from a fixed random teacher).

The reference's client gives every request 5000 ms (kraken/rpc/indep_connecter.h:83-84, not
configurable through its Python API); a pull for a whole 65536-sample batch takes longer than that on
one server and fails with its kTimeoutError.  A global batch is therefore processed the way the
reference is deployed: ``--workers`` independent worker processes (its data parallelism), each running
its share of the batch as forward/backward passes of ``--micro-batch`` samples.

Prints one JSON line with the wall-clock time of the timed steps.
"""
from __future__ import annotations

import argparse
import json
import sys
import time

import numpy as np
import torch

NUM_FIELDS, NUM_DENSE, VOCAB, DIM = 26, 13, 10_000_000, 16
HIDDEN = (400, 400, 400)


def mix64(v: np.ndarray) -> np.ndarray:
    """The 64-bit mixer the benchmark's own data generator uses (only shapes the teacher's features)."""
    u = np.uint64
    with np.errstate(over="ignore"):
        v = v.astype(np.uint64, copy=True)
        v = v * u(3935559000370003845) + u(2691343689449507681)
        v ^= v >> u(21)
        v ^= v << u(37)
        v ^= v >> u(4)
        v *= u(4768777513237032717)
        v ^= v << u(20)
        v ^= v >> u(41)
        v ^= v << u(5)
    return v


def zipf_ids(rng, shape, vocab, s):
    u = rng.random(shape)
    a = 1.0 - s
    r = ((float(vocab + 1) ** a - 1.0) * u + 1.0) ** (1.0 / a) - 1.0
    return np.minimum(r.astype(np.int64), vocab - 1)


class Data:
    def __init__(self, seed):
        self.rng = np.random.default_rng(seed)
        t = np.random.default_rng(12345)
        self.w_dense = t.normal(0.0, 0.1, NUM_DENSE).astype(np.float32)
        self.w_field = t.normal(0.0, 0.1, NUM_FIELDS).astype(np.float32)

    def batch(self, B):
        dense = np.log1p(self.rng.lognormal(0.0, 1.0, (B, NUM_DENSE))).astype(np.float32)
        ids = zipf_ids(self.rng, (B, NUM_FIELDS), VOCAB, 1.1) + (np.arange(NUM_FIELDS, dtype=np.int64) * VOCAB)[None, :]
        h = (mix64(ids.reshape(-1).view(np.uint64)) >> np.uint64(40)).astype(np.float32).reshape(B, NUM_FIELDS)
        h = h / float(1 << 23) - 1.0
        logit = dense @ self.w_dense + h @ self.w_field
        labels = (self.rng.random(B) < 1.0 / (1.0 + np.exp(-logit))).astype(np.float32)
        return torch.from_numpy(dense), torch.from_numpy(ids), torch.from_numpy(labels)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref-path", required=True)
    ap.add_argument("--s-addr", required=True)
    ap.add_argument("--steps", type=int, required=True)
    ap.add_argument("--warmup", type=int, required=True)
    ap.add_argument("--global-batch", type=int, required=True)
    ap.add_argument("--workers", type=int, default=1, help="worker processes sharing every global batch")
    ap.add_argument("--worker-index", type=int, default=0)
    ap.add_argument("--micro-batch", type=int, default=4096,
                    help="samples per forward/backward of one worker (bounded by the reference's 5 s RPC timeout)")
    ap.add_argument("--deadline-s", type=float, default=0.0,
                    help="stop once warm-up plus timed steps have taken this long and report the steps that were finished")
    ap.add_argument("--torch-threads", type=int, default=0)
    args = ap.parse_args()
    if args.torch_threads > 0:
        torch.set_num_threads(args.torch_threads)
    sys.path.insert(0, args.ref_path)
    import kraken.pytorch as kk  # the reference's package

    class DeepFM(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.emb = kk.CombineEmbedding([DIM, 1], initializers=[kk.NormalInitializer(0.0, 0.01),
                                                                    kk.ConstantInitializer(0.0)],
                                           names=["deepfm.second_order", "deepfm.first_order"])
            layers, prev = [], NUM_FIELDS * DIM + NUM_DENSE
            for hdim in HIDDEN:
                layers += [torch.nn.Linear(prev, hdim), torch.nn.ReLU()]
                prev = hdim
            layers.append(torch.nn.Linear(prev, 1))
            self.mlp = torch.nn.Sequential(*layers)

        def forward(self, dense, ids):
            e, w = self.emb([ids, ids])                # [B, F, 16], [B, F, 1]
            s = e.sum(dim=1)
            fm = 0.5 * (s * s - (e * e).sum(dim=1)).sum(dim=1)
            deep = self.mlp(torch.cat([e.flatten(1), dense], dim=1)).squeeze(-1)
            return w.sum(dim=(1, 2)) + fm + deep

    torch.manual_seed(0)
    kk.initialize(args.s_addr)
    model = DeepFM()
    opt = kk.Optimizer("deepfm", model.named_parameters(), 1e-3, kk.Adam(beta1=0.9, beta2=0.999))
    loss_fn = torch.nn.BCEWithLogitsLoss()
    data = Data(1000 + args.worker_index)
    total = args.warmup + args.steps
    share = args.global_batch // args.workers          # this worker's samples of every global batch
    micro = min(args.micro_batch, share)
    n_micro = (share + micro - 1) // micro
    distinct = min(total * n_micro, 64)
    batches = [data.batch(micro) for _ in range(distinct)]

    def micro_step(dense, ids, labels):
        # one forward/backward/step of the reference: pull rows, push sparse and dense gradients (the
        # servers apply every push on arrival), re-pull the dense parameters
        loss = loss_fn(model(dense, ids), labels)
        loss.backward()
        opt.step()
        return float(loss.item())

    last, k = 0.0, 0
    t_begin = time.perf_counter()
    for _ in range(args.warmup):
        for _ in range(n_micro):
            last = micro_step(*batches[k % distinct])
            k += 1
    done = 0
    t0 = time.perf_counter()
    for _ in range(args.steps):
        for _ in range(n_micro):
            last = micro_step(*batches[k % distinct])
            k += 1
        done += 1
        if args.deadline_s > 0 and time.perf_counter() - t_begin > args.deadline_s:
            break
    seconds = time.perf_counter() - t0
    print(json.dumps({"worker": "reference", "index": args.worker_index, "seconds": seconds, "steps": done,
                      "samples": done * n_micro * micro, "micro_batch": micro, "micro_steps_per_step": n_micro,
                      "final_loss": last, "torch_threads": torch.get_num_threads()}), flush=True)
    kk.stop()
    return 0


if __name__ == "__main__":
    sys.exit(main())
