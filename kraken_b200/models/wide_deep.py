"""Wide & Deep on sharded sparse tables.

``WideAndDeep``: single-hot categorical fields; the wide part is a dim-1
embedding per id (summed), the deep part a dim-``dim`` embedding per field
concatenated with the dense features and fed to an MLP - the structure of the
reference's example (examples/WideAndDeep/model.py:60-125), with the hashed
one-hot wide features expressed as a dim-1 table.

``MultiHotWideAndDeep``: every field is a bag of ids (JaggedTensor); all
fields share one combined table keyed by a 64-bit hash, pooled by sum or mean
per field.  On the GPU engine each lookup is one fused pull (dedup, exchange,
gather and pooling) and one fused push.
"""
from __future__ import annotations

from typing import List, Sequence

import torch

from .. import pytorch as kk
from .mlp import MLP


class WideAndDeep(torch.nn.Module):
    def __init__(self, num_fields: int = 26, num_dense: int = 13, dim: int = 8, hidden: Sequence[int] = (256, 128),
                 name: str = "wide_deep", combine: bool = False):
        """``combine``: both tables go through one ``CombineEmbedding`` - one request round per step and direction
        instead of two (what counts on the TCP deployment, where a round is a message to every server)."""
        super().__init__()
        self.num_fields, self.num_dense, self.dim = num_fields, num_dense, dim
        if combine:
            self.both = kk.CombineEmbedding([1, dim], initializers=[kk.ConstantInitializer(0.0),
                                                                    kk.NormalInitializer(0.0, 0.05)],
                                            names=[f"{name}.wide", f"{name}.deep"])
        else:
            self.both = None
            self.wide = kk.Embedding(1, initializer=kk.ConstantInitializer(0.0), name=f"{name}.wide")
            self.deep = kk.Embedding(dim, initializer=kk.NormalInitializer(0.0, 0.05), name=f"{name}.deep")
        width = num_fields * dim + num_dense
        self.mlp_in = (width + 7) // 8 * 8
        self.mlp = MLP(self.mlp_in, list(hidden) + [1])
        self.bias = torch.nn.Parameter(torch.zeros(1))

    def forward(self, dense: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
        if self.both is not None:
            w, e = self.both([ids, ids])
            wide = w.sum(dim=(1, 2))
        else:
            wide = self.wide(ids).sum(dim=(1, 2))
            e = self.deep(ids)
        dense = dense.to(e.device)
        parts = [e.flatten(1), dense]
        if self.mlp_in > e.shape[1] * e.shape[2] + dense.shape[1]:
            parts.append(torch.zeros(dense.shape[0], self.mlp_in - e.shape[1] * e.shape[2] - dense.shape[1],
                                     dtype=e.dtype, device=e.device))
        return wide + self.mlp(torch.cat(parts, dim=1)).squeeze(-1) + self.bias


class MultiHotWideAndDeep(torch.nn.Module):
    """``forward(dense, bags)`` with ``bags`` = one JaggedTensor whose bags are laid out
    sample-major, field-minor: bag ``b * num_fields + f`` holds sample b's ids of field f."""

    def __init__(self, num_fields: int = 100, num_dense: int = 13, dim: int = 64,
                 hidden: Sequence[int] = (1024, 512, 256), mean_fields: Sequence[int] = (), name: str = "mh_wide_deep"):
        super().__init__()
        self.num_fields, self.num_dense, self.dim = num_fields, num_dense, dim
        self.wide = kk.JaggedEmbedding(1, initializer=kk.ConstantInitializer(0.0), name=f"{name}.wide", mode="sum")
        self.deep = kk.Embedding(dim, initializer=kk.NormalInitializer(0.0, 0.05), name=f"{name}.combined")
        mean = torch.zeros(num_fields, dtype=torch.uint8)
        if len(mean_fields):
            mean[list(mean_fields)] = 1
        self.register_buffer("field_is_mean", mean)
        width = num_fields * dim + num_dense
        self.mlp_in = (width + 7) // 8 * 8
        self.mlp = MLP(self.mlp_in, list(hidden) + [1])
        self.bias = torch.nn.Parameter(torch.zeros(1))

    def forward(self, dense: torch.Tensor, bags: kk.JaggedTensor) -> torch.Tensor:
        from ..pytorch import native

        k = bags.num_bags()
        B = k // self.num_fields
        wide = self.wide(bags).view(B, self.num_fields).sum(1)
        tid = self.deep.sparse_table.table_id()
        eng = native.engine()
        if hasattr(eng, "pull_sparse_pooled"):
            bag_mean = self.field_is_mean.repeat(B)
            pooled = _PooledLookup.apply(self.deep.sparse_table, bags.values(), bags.offsets(), bag_mean)
        else:
            emb = self.deep(bags.values())
            off = bags.offsets()
            s = native.jagged_sum_forward(emb, off, 0.0)  # plain CPU path: sum, then scale the mean fields
            lens = (off[1:] - off[:-1]).clamp(min=1).to(s.dtype).unsqueeze(1)
            is_mean = self.field_is_mean.repeat(B).bool().unsqueeze(1)
            pooled = _CpuPool.apply(emb, off, is_mean, lens)
        dense = dense.to(pooled.device)
        parts = [pooled.view(B, self.num_fields * self.dim), dense]
        pad = self.mlp_in - self.num_fields * self.dim - dense.shape[1]
        if pad:
            parts.append(torch.zeros(B, pad, dtype=pooled.dtype, device=pooled.device))
        return wide + self.mlp(torch.cat(parts, dim=1)).squeeze(-1) + self.bias


class _PooledLookup(torch.autograd.Function):
    """Fused bag lookup with a per-bag sum / mean switch (GPU engine)."""

    @staticmethod
    def forward(ctx, sparse_table, values, offsets, bag_mean):
        from ..pytorch import native
        eng = native.engine()
        out, ticket = eng.pull_sparse_pooled(sparse_table.table_id(), values, offsets, bag_mean=bag_mean)
        ctx.state = (eng, sparse_table.table_id(), ticket, values)
        return out

    @staticmethod
    def backward(ctx, grad):
        eng, tid, ticket, values = ctx.state
        eng.push_sparse_pooled(tid, ticket, grad.contiguous(), values)
        return None, None, None, None


class _CpuPool(torch.autograd.Function):
    @staticmethod
    def forward(ctx, emb, offsets, is_mean, lens):
        from ..pytorch import native
        ctx.save_for_backward(offsets, is_mean, lens)
        s = native.jagged_sum_forward(emb, offsets, 0.0)
        return torch.where(is_mean, s / lens, s)

    @staticmethod
    def backward(ctx, grad):
        from ..pytorch import native
        offsets, is_mean, lens = ctx.saved_tensors
        g = torch.where(is_mean, grad / lens, grad).contiguous()
        return native.jagged_sum_backward(offsets, g), None, None, None
