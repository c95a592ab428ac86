#!/usr/bin/env python
"""Headline benchmark: DeepFM training throughput (samples/s) on N GPUs of one box.

Config (the DeepFM configuration of BASELINE.json): 13 dense features, 26
single-hot fields with Zipf(1.1) ids over a vocabulary of 1e7 per field
(2.6e8 possible rows), dim-16 fp32 sparse table + dim-1 first-order table, FM
first/second order + MLP 400-400-400-1, BCE loss, global batch 65536, server
side Adam lr 1e-3.  Synthetic data, random-init weights.

Two timed regions over the same K steps:
  * ``value``  - device time (CUDA events) with the step's inputs already on the device;
  * ``e2e``    - the public API end to end: every step copies its inputs from pinned host
                 memory and reads the loss back.
Multi-GPU runs are launched by torchrun (one rank per GPU); times are the max over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

GLOBAL_BATCH = 65536
NUM_FIELDS, NUM_DENSE, VOCAB, DIM = 26, 13, 10_000_000, 16
HIDDEN = (400, 400, 400)
METRIC = "deepfm_train_samples_per_sec"


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=None,
                   help="timed steps (default: 200 for this framework, 20 for the CPU-bound reference arm)")
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--global-batch", type=int, default=GLOBAL_BATCH)
    p.add_argument("--exchange", default="fused", choices=["fused", "nccl"],
                   help="nccl: the NCCL-only baseline path (implies --no-graph)")
    p.add_argument("--two-tables", action="store_true",
                   help="keep first-order weights in a separate dim-1 table instead of column 16 of the embedding rows")
    p.add_argument("--no-graph", action="store_true", help="launch every kernel from Python instead of replaying a CUDA graph")
    p.add_argument("--no-overlap", action="store_true",
                   help="join the MLP backward's side stream before the sparse backward instead of after the dense step (ablation)")
    p.add_argument("--in-place", action="store_true",
                   help="single GPU: read table rows in place instead of gathering the unique rows (ablation)")
    p.add_argument("--gemm-variant", type=int, default=0,
                   help="MLP GEMM kernel: 0 chosen from the shape, 1 CTA pair, 2 single-CTA resident, 3 tile per CTA (ablation)")
    return p.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "20"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), [c.strip() for c in line.split(",")]))

    def mark(self):
        """Start of the timed regions (device-timed, then end-to-end)."""
        self.t0 = time.perf_counter()

    def stop(self):
        """End of the timed regions.  Samples taken between mark() and now are reported; if the regions
        were shorter than nvidia-smi's period, the samples nearest to them (warm-up steps just before, under
        the same load) are used and ``window`` says so."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        t1 = time.perf_counter()
        time.sleep(0.03)
        self.proc.terminate()
        time.sleep(0.05)
        t0 = getattr(self, "t0", 0.0)
        inside = [r for t, r in self.rows if t0 <= t <= t1 + 0.03]
        window = "timed regions"
        if not inside:
            inside = [r for t, r in self.rows if t0 - 1.0 <= t <= t1 + 0.5]
            window = "nearest samples (regions shorter than the sampling period)"
        self.rows = inside
        sm = sorted(int(r[0]) for r in self.rows if len(r) >= 6 and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) >= 6 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for k, n in enumerate(names) if any(len(r) >= 6 and r[2 + k].lower() == "active" for r in self.rows)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm), "window": window}


def run_ours(args):
    import torch
    import torch.distributed as dist

    import kraken_b200.pytorch as kk
    from kraken_b200.models import ClickDataset, DeepFM
    from kraken_b200.ops import bce_with_logits
    from kraken_b200.utils.prefetch import DevicePrefetcher

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE is {world}: launch with torchrun --nproc-per-node {args.gpus}")
    local_batch = args.global_batch // world
    n_ids = local_batch * NUM_FIELDS
    if args.exchange == "nccl":
        args.no_graph = True
    kk.initialize("gpu", table_capacity=(1 << 26) // world, max_ids_per_call=n_ids, seed=0, exchange=args.exchange,
                  overlap_dense_step=not args.no_overlap)
    dev = torch.device("cuda", torch.cuda.current_device())
    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()  # nvidia-smi takes a second or two to start reporting: launch it ahead of the set-up
    torch.backends.cuda.matmul.allow_tf32 = True
    torch.backends.cudnn.allow_tf32 = True

    if args.gemm_variant:
        from kraken_b200._native import C
        C.gemm_set_tuning(args.gemm_variant, 0)
    torch.manual_seed(0)
    model = DeepFM(NUM_FIELDS, NUM_DENSE, DIM, HIDDEN, fold_first_order=not args.two_tables,
                   in_place_rows=True if args.in_place else None).to(dev)
    opt = kk.Optimizer("deepfm", model.named_parameters(), 1e-3, kk.Adam(beta1=0.9, beta2=0.999))
    eng = kk.native.engine()

    data = ClickDataset(NUM_FIELDS, NUM_DENSE, VOCAB, 1.1, seed=1000 + rank)
    total = args.warmup + args.steps
    # at most 64 distinct batches are generated (1.1 GB of pinned ids at batch 65536); longer runs cycle through them
    distinct = min(total, 64)
    host = [data.batch(local_batch, pin=True) for _ in range(distinct)]
    h2d_bytes = sum(t.numel() * t.element_size() for t in host[0])
    inv_world = 1.0 / world  # local mean * 1/world summed over ranks = global mean

    def eager_step(dense, ids, labels):
        logits = model(dense, ids)
        loss = bce_with_logits(logits, labels)
        if world > 1:
            loss = loss * inv_world
        loss.backward()
        opt.step()
        return loss

    staged0 = tuple(t.to(dev) for t in host[0])
    if args.no_graph:
        step = eager_step
    else:
        from kraken_b200.utils.graph import GraphedStep
        l0 = eng.kernel_launches()
        eager_step(*staged0)  # first call: collective set-up of channels and bucket
        l1 = eng.kernel_launches()
        eager_step(*staged0)
        launches_per_step = eng.kernel_launches() - l1
        step = GraphedStep(eager_step, staged0, warmup=2, slots=2)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---------------- device-timed region: inputs staged on the device beforehand
    staged = [tuple(t.to(dev, non_blocking=True) for t in b) for b in host]
    for i in range(args.warmup):
        step(*staged[i % distinct])
    eng.check()
    launches0 = eng.kernel_launches()
    sync_all()
    sampler.mark()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.warmup, total):
        step(*staged[i % distinct])
    e1.record()
    sync_all()
    dev_ms = max_over_ranks(e0.elapsed_time(e1))
    launches = eng.kernel_launches() - launches0
    if not args.no_graph:
        launches = launches_per_step * args.steps  # replayed from the graph: counted once at capture
    eng.check()

    # ---------------- end-to-end region: pinned host inputs in, loss out, every step
    for batch in DevicePrefetcher((host[i % distinct] for i in range(min(3, args.warmup))), dev):
        step(*batch).item()
    sync_all()
    t0 = time.perf_counter()
    e0.record()
    last = 0.0
    # batch i+1 crosses PCIe on a copy stream while batch i trains; every copy is inside the timed region
    # and the loss of step i is read back after step i+1 has been enqueued, so the device does not wait for the host
    pending = None
    loader = (host[i % distinct] for i in range(args.warmup, total))
    if args.no_graph:
        for batch in DevicePrefetcher(loader, dev):
            last = step(*batch).item()
    else:
        # the prefetcher writes straight into the input buffers of the graph that runs next (two graphs, two sets)
        pf = DevicePrefetcher(loader, dev, buffers=[step.static_inputs(0), step.static_inputs(1)])
        for _ in pf:
            handle = step.launch_slot(pf.last_slot)
            if pending is not None:
                last = pending.item()
            pending = handle
    if pending is not None:
        last = pending.item()
    e1.record()
    sync_all()
    e2e_ms = max_over_ranks(max(e0.elapsed_time(e1), (time.perf_counter() - t0) * 1e3 if world == 1 else 0.0))
    clocks = sampler.stop()  # samples cover the device-timed and the end-to-end region
    eng.check()

    if rank == 0:
        value = args.global_batch * args.steps / (dev_ms / 1e3)
        out = {
            "metric": METRIC, "value": value, "unit": "samples/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": dev_ms / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            # bf16 is the LOWEST precision of any stage; what each stage runs in:
            "precision": {"tables_and_row_optimizer": "fp32", "fm_interaction_logit_loss": "fp32",
                          "mlp_gemm_operands": "bf16, fp32 accumulation (TMEM), fp32 master weights",
                          "mlp_input_gradient_dx": "bf16", "weight_gradients_and_dense_optimizer": "fp32",
                          "parity_with_fp32": "python -m kraken_b200.benchmarks.precision_parity prints loss and AUC of both"},
            "impl": "ours" if args.exchange == "fused" else "ours-nccl-baseline",
            "config": {"model": "DeepFM 26x1e7 dim16 + MLP 400-400-400-1, Adam lr 1e-3",
                       "tables": "dim-16 embedding + dim-1 first-order" if args.two_tables else
                       "one table, rows = 16 embedding floats + first-order weight (padded to 20)", "global_batch": args.global_batch,
                       "seq_len": NUM_FIELDS, "parallelism": f"dp{world}+row-sharded-tables{world}",
                       "launch": "eager" if args.no_graph else "cuda-graph replay of the whole step",
                       "l2": "working set (hash-table rows touched per step + slabs) exceeds the 126 MB L2; "
                             "a different batch every step (64 distinct batches, cycled)"},
            "clocks": clocks,
            "e2e": {"value": args.global_batch * args.steps / (e2e_ms / 1e3), "unit": "samples/s",
                    "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": 4, "ms_per_step": e2e_ms / args.steps},
            "gpu_launches": launches, "final_loss": last * world,
        }
        print(json.dumps(out), flush=True)
    kk.stop()


def run_reference(args):
    from baseline.reference_arm import run
    run(args)


if __name__ == "__main__":
    a = parse()
    if a.steps is None:
        a.steps = 20 if a.impl == "reference" else 200
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
