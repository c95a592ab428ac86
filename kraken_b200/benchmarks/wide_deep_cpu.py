"""Wide&Deep on the CPU engine: 1 shard + 1 worker in one process, fp32, 200 steps, batch 512,
26 single-hot fields with Zipf(1.05) ids over 1e5 per field, server-side Adagrad lr 0.01 with
initial accumulator 0.1.  Prints train samples/s.

    python -m kraken_b200.benchmarks.wide_deep_cpu [--steps 200]
"""
import argparse
import time

import torch

import kraken_b200.pytorch as kk
from kraken_b200.benchmarks.common import emit
from kraken_b200.models import ClickDataset, WideAndDeep
from kraken_b200.ops import bce_with_logits


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--steps", type=int, default=200)
    p.add_argument("--batch", type=int, default=512)
    a = p.parse_args()
    torch.manual_seed(0)
    kk.initialize("cpu", seed=0)
    model = WideAndDeep(26, 13, 8, (256, 128))
    opt = kk.Optimizer("wide_deep", model.named_parameters(), 0.01, kk.Adagrad(initial_accumulator_value=0.1))
    data = ClickDataset(26, 13, 100_000, 1.05, seed=0)
    batches = [data.batch(a.batch) for _ in range(a.steps)]
    losses = []
    t0 = time.perf_counter()
    for dense, ids, labels in batches:
        loss = bce_with_logits(model(dense, ids), labels)
        loss.backward()
        opt.step()
        losses.append(loss.item())
    dt = time.perf_counter() - t0
    emit({"benchmark": "wide_deep_cpu", "engine": "cpu", "steps": a.steps, "batch": a.batch,
          "samples_per_sec": a.steps * a.batch / dt, "ms_per_step": dt / a.steps * 1e3,
          "loss_first10": sum(losses[:10]) / 10, "loss_last10": sum(losses[-10:]) / 10})
    kk.stop()


if __name__ == "__main__":
    main()
