"""Dense-table path: MLP 784-4096-4096-4096-10 (ReLU, cross entropy) on synthetic 28x28 images,
batch 1024 per GPU, server-side SGD momentum 0.9 lr 0.05, with or without DCT gradient
compression (keeps the top 25 % by magnitude, threshold refreshed every 1000 steps).

    torchrun --nproc-per-node N -m kraken_b200.benchmarks.dense_dct [--dct] [--steps 30]
"""
import argparse
import re

import numpy as np
import torch

import kraken_b200.pytorch as kk
from kraken_b200.benchmarks.common import DeviceTimer, emit, measure_copy_gbs, measure_peer_gbs, world_rank
from kraken_b200.models import MLP, mnist_like


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--steps", type=int, default=30)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--batch", type=int, default=1024)
    p.add_argument("--dct", action="store_true")
    p.add_argument("--no-overlap", action="store_true",
                   help="step all buckets after the backward pass instead of each as soon as its gradients exist")
    p.add_argument("--graph", action="store_true", help="replay the training step as one CUDA graph (not with --dct)")
    p.add_argument("--timeline", action="store_true",
                   help="also print rank 0's per-kernel timeline of one fused dense step (start, duration, kernel), taken "
                        "with torch.profiler - for diagnosis, never a benchmark number")
    a = p.parse_args()
    world, rank = world_rank()
    kk.initialize("gpu", emitter_type=kk.EmitterType.kDCT if a.dct else kk.EmitterType.kDefault, life_span=1000,
                  eta=0.75, overlap_dense_step=not a.no_overlap)
    dev = torch.device("cuda", torch.cuda.current_device())
    torch.manual_seed(0)
    model = MLP(784, [4096, 4096, 4096, 10]).to(dev)
    opt = kk.Optimizer("mnist_mlp", model.named_parameters(), 0.05, kk.SGD(momentum=0.9))
    rng = np.random.default_rng(100 + rank)
    means = np.random.default_rng(7).normal(0, 1, (10, 784)).astype(np.float32)
    total = a.warmup + a.steps
    batches = [tuple(t.to(dev) for t in mnist_like(rng, means, a.batch)) for _ in range(total)]
    scale = 1.0 / world

    def eager_step(x, y):
        loss = torch.nn.functional.cross_entropy(model(x), y) * scale
        loss.backward()
        opt.step()
        return loss

    step = eager_step
    if a.graph and not a.dct:
        from kraken_b200.utils.graph import GraphedStep
        step = GraphedStep(eager_step, batches[0], warmup=2, optimizer=None)

    for i in range(a.warmup):
        step(*batches[i])
    kk.native.engine().check()
    timer = DeviceTimer()
    timer.start()
    for i in range(a.warmup, total):
        loss = step(*batches[i])
    ms = timer.stop_ms()
    kk.native.engine().check()
    n_params = sum(p.numel() for p in model.parameters())
    rec = {"benchmark": "dense_mlp" + ("_dct" if a.dct else ""), "n_gpus": world, "batch_per_gpu": a.batch,
           "params": n_params, "samples_per_sec": a.batch * world * a.steps / (ms / 1e3), "ms_per_step": ms / a.steps,
           "final_loss": loss.item() * world, "dense_step": "all buckets after backward" if a.no_overlap else
           "each bucket as soon as its gradients exist", "launch": "cuda-graph replay" if (a.graph and not a.dct) else "eager",
           "buckets": len(kk.native.engine().bucket.buckets) if getattr(kk.native.engine(), "bucket", None) else 0}

    # the fused dense step alone (reduce-scatter + optimizer + all-gather in one kernel), on whatever the
    # gradient buffer holds; every rank starts each step together (the timer synchronises and barriers)
    eng = kk.native.engine()
    if not a.dct and getattr(eng, "bucket", None) is not None:
        for _ in range(3):
            eng.dense_step()
        step_ms = 0.0
        for _ in range(10):
            timer.start()
            eng.dense_step()
            step_ms += timer.stop_ms()
        us_eager = step_ms / 10 * 1e3
        # the same call as one CUDA-graph replay: what it costs inside a captured training step, without the
        # host's launch overhead between its short kernels
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            eng.dense_step()
        for _ in range(3):
            g.replay()
        step_ms = 0.0
        for _ in range(10):
            timer.start()
            g.replay()
            step_ms += timer.stop_ms()
        us = step_ms / 10 * 1e3
        n_pad = int(eng.bucket.n_pad)
        # per GPU and direction, (G - 1) / G of the bucket crosses the link TWICE: inbound are the peers' gradient
        # slices this owner loads AND the other owners' weight slices stored into this rank's copy; outbound the
        # mirror image (this rank's gradient read by the other owners, its own slice stored to every peer)
        link = 2 * (world - 1) / world * n_pad * 4
        # HBM: G gradient slices read + zeroed bucket, owned slice of value and momentum read + written,
        # the whole updated bucket written once by the owners
        hbm = n_pad * 4 * (1 + 1 + 1) + (n_pad / world) * 4 * 4
        hbm_gbs, link_gbs = measure_copy_gbs(dev), measure_peer_gbs()
        link_us, hbm_us = (link / (link_gbs * 1e3) if link_gbs > 0 else 0.0), hbm / (hbm_gbs * 1e3)
        rec.update({"dense_step_us": round(us, 1), "dense_step_eager_us": round(us_eager, 1),
                    "hbm_copy_gbs": round(hbm_gbs, 1), "peer_copy_gbs_per_direction": round(link_gbs, 1),
                    "dense_step_nvlink_bound_us": round(link_us, 1),
                    "dense_step_hbm_bound_us": round(hbm_us, 1),
                    "dense_step_roofline_fraction": round(max(link_us, hbm_us) / us, 3)})
    if a.timeline and not a.dct and getattr(eng, "bucket", None) is not None:
        from torch.profiler import ProfilerActivity, profile
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for _ in range(3):
                timer.start()          # barrier + synchronize: every rank enters the step together
                eng.dense_step()
                torch.cuda.synchronize()
        if rank == 0:
            evs = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA and "dense_" in e.name),
                         key=lambda e: e.time_range.start)
            last = evs[-(len(evs) // 3):]
            t0 = last[0].time_range.start
            rec["dense_step_timeline_us"] = [[round(e.time_range.start - t0, 1), round(e.time_range.end - e.time_range.start, 1),
                                              re.search(r"dense_\w+(<[^>]*>)?", e.name).group(0)] for e in last]
    emit(rec)
    kk.stop()


if __name__ == "__main__":
    main()
