"""Multi-hot Wide&Deep: F fields share one combined dim-64 table keyed by a 2^40 hash; bag
lengths ~ Poisson(20) clipped to [1, 100]; sum pooling, mean for half of the fields; deep MLP
1024-512-256-1; server-side Adagrad.  Exercises dedup, pooled gather and segment-sum push.

    torchrun --nproc-per-node N -m kraken_b200.benchmarks.multihot [--batch 16384] [--fields 100]
"""
import argparse

import torch

import kraken_b200.pytorch as kk
from kraken_b200.benchmarks.common import DeviceTimer, emit, world_rank
from kraken_b200.models import MultiHotDataset, MultiHotWideAndDeep
from kraken_b200.ops import bce_with_logits


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--steps", type=int, default=10)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--batch", type=int, default=16384)
    p.add_argument("--fields", type=int, default=100)
    p.add_argument("--vocab", type=int, default=(1 << 40) // 100,
                   help="Zipf ranks per field; (field, rank) is hashed into the 2^40 id space (default: the fields "
                        "together span all of it)")
    p.add_argument("--table-capacity", type=int, default=1 << 27, help="initial slots per GPU shard")
    a = p.parse_args()
    world, rank = world_rank()
    max_ids = int(a.batch * a.fields * 21.5)
    max_unique = max(1 << 20, max_ids // 2)
    kk.initialize("gpu", table_capacity=a.table_capacity, max_ids_per_call=max_ids, max_unique_per_call=max_unique,
                  max_per_owner_per_call=max_unique if world == 1 else int(2.5 * max_unique / world))
    dev = torch.device("cuda", torch.cuda.current_device())
    torch.manual_seed(0)
    model = MultiHotWideAndDeep(a.fields, 13, 64, (1024, 512, 256), mean_fields=range(0, a.fields, 2)).to(dev)
    opt = kk.Optimizer("multihot", model.named_parameters(), 0.01, kk.Adagrad(initial_accumulator_value=0.1))
    data = MultiHotDataset(a.fields, 13, a.vocab, 1.1, seed=10 + rank)
    total = a.warmup + a.steps
    batches = [[t.to(dev) for t in data.batch(a.batch)] for _ in range(total)]
    scale = 1.0 / world

    def step(dense, ids, offsets, labels):
        loss = bce_with_logits(model(dense, kk.JaggedTensor(ids, offsets, validate=False)), labels) * scale
        loss.backward()
        opt.step()
        return loss

    for i in range(a.warmup):
        step(*batches[i])
    kk.native.engine().check()
    timer = DeviceTimer()
    timer.start()
    for i in range(a.warmup, total):
        loss = step(*batches[i])
    ms = timer.stop_ms()
    kk.native.engine().check()
    ids_per_step = sum(int(b[1].numel()) for b in batches[a.warmup:]) / a.steps
    emit({"benchmark": "multihot_wide_deep", "n_gpus": world, "batch_per_gpu": a.batch, "fields": a.fields,
          "ids_per_gpu_step": ids_per_step, "samples_per_sec": a.batch * world * a.steps / (ms / 1e3),
          "ms_per_step": ms / a.steps, "final_loss": loss.item() * world, "id_space": "2^40 (hashed Zipf ranks)",
          "ranks_per_field": a.vocab, "rows_per_gpu_after": sum(t.num_rows() for t in kk.native.engine().sparse.values())})
    kk.stop()


if __name__ == "__main__":
    main()
