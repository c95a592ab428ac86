"""Wide & Deep with ONE table per categorical field, looked up through the combined calls.

The reference reserves examples/WideAndDeep_Combine for this demo but ships only empty files
(examples/WideAndDeep_Combine/*.py are 0 bytes).  Here every field owns a dim-1 "wide" table and a
dim-``--dim`` "deep" table - the layout of the reference's DeepFM example, 2 x F small tables
(examples/DeepFM/model/DeepFM.py:64-69) - and the model asks for all of them in one
``kk.CombineEmbedding`` call: on the GPU engine that is one exchange per row width (two in all) instead
of 2 x F, on the TCP deployment one request round per server (kraken/worker/emitter.cc:185-278).

    python examples/wide_deep_combine/main.py [--s_addr cpu|gpu|tcp://host:port] [--fields 13]
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import kraken_b200.pytorch as kk  # noqa: E402
from kraken_b200.models import ClickDataset  # noqa: E402
from kraken_b200.models.mlp import MLP  # noqa: E402
from kraken_b200.ops import bce_with_logits  # noqa: E402


class CombinedWideAndDeep(torch.nn.Module):
    def __init__(self, fields: int, num_dense: int, dim: int, hidden):
        super().__init__()
        self.fields, self.dim = fields, dim
        self.tables = kk.CombineEmbedding(
            dimensions=[1] * fields + [dim] * fields,
            initializers=[kk.ConstantInitializer(0.0)] * fields + [kk.NormalInitializer(0.0, 0.05)] * fields,
            names=[f"wide.{f}" for f in range(fields)] + [f"deep.{f}" for f in range(fields)])
        width = fields * dim + num_dense
        self.mlp_in = (width + 7) // 8 * 8
        self.mlp = MLP(self.mlp_in, list(hidden) + [1])

    def forward(self, dense, ids):
        # ids [B, F] are local to their field: every field has its own pair of tables
        cols = [ids[:, f].contiguous() for f in range(self.fields)]
        rows = self.tables(cols + cols)
        wide = torch.stack([r.squeeze(-1) for r in rows[:self.fields]], dim=1).sum(dim=1)
        deep = torch.cat(rows[self.fields:], dim=1)
        parts = [deep, dense.to(deep.device)]
        pad = self.mlp_in - deep.shape[1] - dense.shape[1]
        if pad:
            parts.append(torch.zeros(deep.shape[0], pad, dtype=deep.dtype, device=deep.device))
        return wide + self.mlp(torch.cat(parts, dim=1)).squeeze(-1)


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--s_addr", default="auto")
    p.add_argument("--steps", type=int, default=100)
    p.add_argument("--batch", type=int, default=512)
    p.add_argument("--fields", type=int, default=13)
    p.add_argument("--dim", type=int, default=8)
    a = p.parse_args()
    kk.initialize(a.s_addr)
    eng = kk.native.engine()
    dev = eng.device
    torch.manual_seed(0)
    model = CombinedWideAndDeep(a.fields, 13, a.dim, (128, 64)).to(dev)
    opt = kk.Optimizer("wide_deep_combine", model.named_parameters(), 0.01, kk.Adagrad(initial_accumulator_value=0.1))
    data = ClickDataset(a.fields, 13, 50_000, 1.05, seed=eng.rank)
    vocab_base = torch.arange(a.fields, dtype=torch.int64) * 50_000
    first = last = None
    for step in range(a.steps):
        dense, ids, labels = data.batch(a.batch)
        ids = ids - vocab_base            # back to per-field ids
        dense, ids, labels = dense.to(dev), ids.to(dev), labels.to(dev)
        loss = bce_with_logits(model(dense, ids), labels) / eng.world
        loss.backward()
        opt.step()
        if step % 20 == 0 or step == a.steps - 1:
            last = loss.item() * eng.world
            first = last if first is None else first
            if eng.rank == 0:
                print(f"step {step:4d}  loss {last:.4f}")
    if eng.rank == 0:
        print(f"done: {2 * a.fields} tables, loss {first:.4f} -> {last:.4f}")
    kk.stop()


if __name__ == "__main__":
    main()
