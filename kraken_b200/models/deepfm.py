"""DeepFM on sharded sparse tables.

One dim-``dim`` table holds the second-order / deep embeddings of all fields
and one dim-1 table the first-order weights; ids are global (field offset
already added).  logit = sum_f w_f + FM2(e) + MLP([e, dense]) + bias.  The
reference's example builds the same model from 39 + 39 small tables and torch
CPU ops (examples/DeepFM/model/DeepFM.py:64-140).
"""
from __future__ import annotations

from typing import Sequence

import torch

from .. import pytorch as kk
from ..ops import fm_interaction
from .mlp import MLP


class DeepFM(torch.nn.Module):
    def __init__(self, num_fields: int = 26, num_dense: int = 13, dim: int = 16,
                 hidden: Sequence[int] = (400, 400, 400), init_std: float = 0.01, name: str = "deepfm"):
        super().__init__()
        self.num_fields, self.num_dense, self.dim = num_fields, num_dense, dim
        self.first_order = kk.Embedding(1, initializer=kk.ConstantInitializer(0.0), name=f"{name}.first_order")
        self.second_order = kk.Embedding(dim, initializer=kk.NormalInitializer(0.0, init_std),
                                         name=f"{name}.second_order")
        self.mlp = MLP(num_fields * dim + num_dense, list(hidden) + [1])
        self.bias = torch.nn.Parameter(torch.zeros(1))

    def forward(self, dense: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
        w = self.first_order(ids)       # [B, F, 1]
        e = self.second_order(ids)      # [B, F, dim]
        dense = dense.to(e.device)
        deep = self.mlp(torch.cat([e.flatten(1), dense], dim=1)).squeeze(-1)
        return w.sum(dim=(1, 2)) + fm_interaction(e) + deep + self.bias
