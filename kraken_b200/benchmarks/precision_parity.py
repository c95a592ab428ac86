"""Precision parity of the benchmark's DeepFM step: fused bf16 path against an all-fp32 path.

The reference computes everything in fp32 (kraken/t/math.cc:20-76; its example model is plain torch
CPU ops, examples/DeepFM/model/DeepFM.py:96-116).  The headline step of this framework keeps tables,
optimizer state, accumulators and master weights in fp32 but feeds the MLP's tensor-core GEMMs with
bf16 operands and carries the MLP-input gradient in bf16.  This script trains the SAME model on the
SAME batches twice on one GPU -

    arm "bf16"  : the fused front end + tcgen05 MLP, exactly what bench.py times;
    arm "fp32"  : DeepFM(fused=False) with torch fp32 matmuls (TF32 off), embeddings expanded to
                  [B, F, dim] fp32 tensors, the unfused pull / push;

- and reports, for each, the training loss over the last 100 steps and loss + AUC on held-out batches of
the same teacher task.  One JSON line.

    python -m kraken_b200.benchmarks.precision_parity [--steps 2048] [--batch 65536]
"""
import argparse
import time

import torch

import kraken_b200.pytorch as kk
from kraken_b200.benchmarks.common import emit
from kraken_b200.models import ClickDataset, DeepFM
from kraken_b200.ops import bce_with_logits


def auc(logits: torch.Tensor, labels: torch.Tensor) -> float:
    """Area under the ROC curve by the rank statistic (ties are rare in fp32 logits)."""
    order = torch.argsort(logits)
    ranks = torch.empty_like(order, dtype=torch.float64)
    ranks[order] = torch.arange(1, logits.numel() + 1, device=logits.device, dtype=torch.float64)
    pos = labels > 0.5
    n_pos, n_neg = int(pos.sum()), int((~pos).sum())
    if n_pos == 0 or n_neg == 0:
        return float("nan")
    return float((ranks[pos].sum() - n_pos * (n_pos + 1) / 2) / (n_pos * n_neg))


class DeviceClickData:
    """The benchmark's synthetic task generated on the device, so that thousands of DISTINCT batches cost
    nothing on the host: log1p(LogNormal) dense features, Zipf(s) ids per field (inverse CDF of the continuous
    envelope, as the host generator), labels ~ Bernoulli(sigmoid(teacher)) with the teacher linear in the dense
    features and in a pseudo-random feature of every (field, id).  Same seed -> same stream, on every run."""

    def __init__(self, fields: int, num_dense: int, vocab: int, s: float, seed: int, dev):
        self.F, self.D, self.vocab, self.s, self.dev = fields, num_dense, vocab, s, dev
        self.gen = torch.Generator(device=dev).manual_seed(seed)
        t = torch.Generator().manual_seed(12345)
        # a stronger teacher than the timing benchmark's (std 0.5): the task must be learnable in 2k steps
        self.w_dense = (torch.randn(num_dense, generator=t) * 0.5).to(dev)
        self.w_field = (torch.randn(fields, generator=t) * 0.5).to(dev)
        self.base = (torch.arange(fields, dtype=torch.int64) * vocab).to(dev)

    def batch(self, B: int):
        dense = torch.log1p(torch.exp(torch.randn(B, self.D, generator=self.gen, device=self.dev)))
        u = torch.rand(B, self.F, generator=self.gen, device=self.dev, dtype=torch.float64)
        a = 1.0 - self.s
        r = ((float(self.vocab + 1) ** a - 1.0) * u + 1.0) ** (1.0 / a) - 1.0
        ids = r.to(torch.int64).clamp_(max=self.vocab - 1) + self.base
        h = ((ids * 0x9E3779B97F4A7C15) >> 40) & 0xFFFFFF          # 24 pseudo-random bits per (field, id)
        h = h.to(torch.float32) / float(1 << 23) - 1.0
        logit = dense @ self.w_dense + h @ self.w_field - float(self.w_dense.sum()) * 0.8
        labels = (torch.rand(B, generator=self.gen, device=self.dev) < torch.sigmoid(logit)).to(torch.float32)
        return dense, ids, labels


def run_arm(fused: bool, batches, evals, a, dev) -> dict:
    kk.initialize("gpu", table_capacity=a.table_capacity, max_ids_per_call=a.batch * a.fields, seed=0)
    torch.manual_seed(0)
    model = DeepFM(a.fields, 13, 16, (400, 400, 400), fused=fused, fold_first_order=True).to(dev)  # same table layout in both arms
    if not fused:
        model.mlp.use_tensor_cores = False
    opt = kk.Optimizer("deepfm", model.named_parameters(), 1e-3, kk.Adam(beta1=0.9, beta2=0.999))
    eng = kk.native.engine()
    losses = []
    t0 = time.perf_counter()
    stream = DeviceClickData(a.fields, 13, a.vocab, 1.1, 1000, dev) if batches is None else None
    for s in range(a.steps):
        if stream is not None:
            dense, ids, labels = stream.batch(a.batch)   # a new batch every step, the same sequence in both arms
        else:
            dense, ids, labels = (t.to(dev, non_blocking=True) for t in batches[s % len(batches)])
        loss = bce_with_logits(model(dense, ids), labels)
        loss.backward()
        opt.step()
        if s >= a.steps - 100:
            losses.append(loss.detach())
    torch.cuda.synchronize()
    train_s = time.perf_counter() - t0
    eng.check()
    logits, labels_all = [], []
    with torch.no_grad():
        for dense, ids, labels in evals:
            logits.append(model(dense.to(dev), ids.to(dev)).float())
            labels_all.append(labels.to(dev))
    logits, labels_all = torch.cat(logits), torch.cat(labels_all)
    out = {"train_loss_last100": float(torch.stack(losses).mean()),
           "eval_loss": float(torch.nn.functional.binary_cross_entropy_with_logits(logits, labels_all)),
           "eval_auc": auc(logits, labels_all), "train_seconds": round(train_s, 2),
           "rows": sum(t.num_rows() for t in eng.sparse.values())}
    kk.stop()
    return out


def main(argv=None) -> dict:
    p = argparse.ArgumentParser()
    p.add_argument("--steps", type=int, default=2048)
    p.add_argument("--batch", type=int, default=65536)
    p.add_argument("--fields", type=int, default=26)
    p.add_argument("--vocab", type=int, default=10_000_000)
    p.add_argument("--distinct", type=int, default=0,
                   help="0 (default): every step trains on a NEW batch generated on the device; n > 0: n distinct "
                        "batches of the host generator, cycled (the model then memorises them)")
    p.add_argument("--eval-batches", type=int, default=8)
    p.add_argument("--table-capacity", type=int, default=1 << 27)
    a = p.parse_args(argv)
    dev = torch.device("cuda", torch.cuda.current_device())
    torch.backends.cuda.matmul.allow_tf32 = False  # the fp32 arm is real fp32
    torch.backends.cudnn.allow_tf32 = False
    if a.distinct > 0:
        data = ClickDataset(a.fields, 13, a.vocab, 1.1, seed=1000)
        batches = [data.batch(a.batch, pin=True) for _ in range(min(a.distinct, a.steps))]
        held_out = ClickDataset(a.fields, 13, a.vocab, 1.1, seed=77)
        evals = [held_out.batch(a.batch) for _ in range(a.eval_batches)]
    else:
        batches = None
        held_out = DeviceClickData(a.fields, 13, a.vocab, 1.1, 77, dev)
        evals = [held_out.batch(a.batch) for _ in range(a.eval_batches)]
    rec = {"benchmark": "precision_parity", "model": "DeepFM 26x1e7 dim16 + MLP 400-400-400-1, Adam lr 1e-3",
           "steps": a.steps, "batch": a.batch,
           "data": "a new batch every step (device generator)" if batches is None else f"{len(batches)} host batches, cycled",
           "stages_bf16_arm": {"tables_and_optimizer_state": "fp32", "fm_logit_and_loss": "fp32",
                               "mlp_operands": "bf16 (fp32 accumulation in TMEM, fp32 master weights)",
                               "mlp_input_gradient": "bf16", "dense_optimizer": "fp32"}}
    rec["bf16"] = run_arm(True, batches, evals, a, dev)
    rec["fp32"] = run_arm(False, batches, evals, a, dev)
    rec["eval_loss_diff"] = rec["bf16"]["eval_loss"] - rec["fp32"]["eval_loss"]
    rec["eval_auc_diff"] = rec["bf16"]["eval_auc"] - rec["fp32"]["eval_auc"]
    emit(rec)
    return rec


if __name__ == "__main__":
    main()
