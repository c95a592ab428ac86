"""Embedding lookups backed by sharded sparse tables.

forward = sparse pull (rows of unseen ids are created by the table's
initializer), backward = sparse push (duplicate ids summed, optimizer applied
on the owning shard).  Nothing flows back into autograd for the table itself
(kraken/pytorch/embedding.py:9-42, kraken/pytorch/combine_embedding.py:10-52).
"""
from typing import List, Optional

import torch

from . import native
from .initializer import Initializer
from .sparse_table import CombineSparseTable, SparseTable


class EmbeddingFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, sparse_table, indices):
        ctx.table_id = sparse_table.table_id()
        if ctx.table_id is None:
            raise native.KrakenError("the sparse table is not registered: build kraken's Optimizer first")
        ctx.indices = indices
        return native.pull_sparse_table(ctx.table_id, indices)

    @staticmethod
    def backward(ctx, grad):
        native.push_sparse_table(ctx.table_id, ctx.indices, grad)
        return None, None


class Embedding(torch.nn.Module):
    def __init__(self, dimension: int, dtype: torch.dtype = torch.float32, initializer: Optional[Initializer] = None,
                 name: Optional[str] = None):
        super().__init__()
        self.sparse_table = SparseTable(dimension=dimension, dtype=dtype, initializer=initializer, name=name)

    def forward(self, indices):
        return EmbeddingFunction.apply(self.sparse_table, indices)


class CombineEmbeddingFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, combine_sparse_table, *indices):
        ctx.table_ids = combine_sparse_table.table_ids()
        if ctx.table_ids is None:
            raise native.KrakenError("the sparse tables are not registered: build kraken's Optimizer first")
        ctx.indices = list(indices)
        return tuple(native.combine_pull_sparse_table(ctx.table_ids, ctx.indices))

    @staticmethod
    def backward(ctx, *grads):
        native.combine_push_sparse_table(ctx.table_ids, ctx.indices, list(grads))
        return (None,) * (1 + len(grads))


class CombineEmbedding(torch.nn.Module):
    """N tables looked up by one call: ``forward(List[Tensor]) -> List[Tensor]``."""

    def __init__(self, dimensions: List[int], dtypes: Optional[List[torch.dtype]] = None,
                 initializers: Optional[List[Initializer]] = None, names: Optional[List[str]] = None):
        super().__init__()
        self.combine_sparse_table = CombineSparseTable(dimensions=dimensions, dtypes=dtypes,
                                                       initializers=initializers, names=names)

    def forward(self, indices: List[torch.Tensor]):
        if len(indices) != len(self.combine_sparse_table.dimensions()):
            raise ValueError("one index tensor per table is required")
        return list(CombineEmbeddingFunction.apply(self.combine_sparse_table, *indices))
