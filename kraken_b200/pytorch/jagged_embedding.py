"""EmbeddingBag over a sharded sparse table: lookup, optional per-id weights,
then sum or mean pooling per bag, empty bags yielding ``patch_value``
(kraken/pytorch/jagged_embedding.py:10-52, combine_jagged_embedding.py:11-76).
On the GPU engine lookup and pooling are one fused operation."""
from typing import List, Optional

import torch

from . import native
from .embedding import CombineEmbedding, Embedding
from .initializer import Initializer
from .jagged_embedding_funcs import (FusedCombineJaggedLookupFunction, FusedJaggedLookupFunction,
                                     JaggedEmbeddingMeanFunction, JaggedEmbeddingSumFunction)
from .jagged_tensor import JaggedTensor

_MODES = ("sum", "mean")


def _pool(embeddings, offsets, weights, mode, patch_value):
    if weights is not None:
        embeddings = embeddings * weights.unsqueeze(-1)
    fn = JaggedEmbeddingSumFunction if mode == "sum" else JaggedEmbeddingMeanFunction
    return fn.apply(embeddings, offsets.to(embeddings.device), patch_value)


def _fused_available() -> bool:
    return (native.is_initialized() and hasattr(native.engine(), "pull_sparse_pooled")
            and not getattr(native.engine(), "nccl", False))


class JaggedEmbedding(torch.nn.Module):
    def __init__(self, dimension: int, dtype: torch.dtype = torch.float32, initializer: Optional[Initializer] = None,
                 name: Optional[str] = None, mode: str = "sum", patch_value: float = 0.0):
        super().__init__()
        if mode not in _MODES:
            raise ValueError("JaggedEmbedding's mode only supports sum/mean")
        self.embedding = Embedding(dimension=dimension, dtype=dtype, initializer=initializer, name=name)
        self._mode = mode
        self._patch_value = float(patch_value)

    def forward(self, input: JaggedTensor):
        if _fused_available() and input.values().dim() == 1:
            return FusedJaggedLookupFunction.apply(self.embedding.sparse_table, input.values(), input.offsets(),
                                                   input.weights(), self._mode == "mean", self._patch_value)
        emb = self.embedding(input.values())
        return _pool(emb, input.offsets(), input.weights(), self._mode, self._patch_value)


class CombineJaggedEmbedding(torch.nn.Module):
    def __init__(self, dimensions: List[int], dtypes: Optional[List[torch.dtype]] = None,
                 initializers: Optional[List[Initializer]] = None, names: Optional[List[str]] = None,
                 modes: Optional[List[str]] = None, patch_values: Optional[List[float]] = None):
        super().__init__()
        n = len(dimensions)
        if modes is not None:
            if len(modes) != n or any(m not in _MODES for m in modes):
                raise ValueError("CombineJaggedEmbedding needs one mode (sum/mean) per table")
        if patch_values is not None and len(patch_values) != n:
            raise ValueError("CombineJaggedEmbedding needs one patch value per table")
        self.combine_embedding = CombineEmbedding(dimensions=dimensions, dtypes=dtypes, initializers=initializers,
                                                  names=names)
        self._modes = list(modes) if modes is not None else ["sum"] * n
        self._patch_values = [float(p) for p in patch_values] if patch_values is not None else [0.0] * n

    def forward(self, inputs: List[JaggedTensor]):
        if len(inputs) != len(self._modes):
            raise ValueError("one JaggedTensor per table is required")
        if (_fused_available() and hasattr(native.engine(), "combine_pull_sparse_pooled")
                and all(i.values().dim() == 1 for i in inputs)):
            outs = FusedCombineJaggedLookupFunction.apply(
                self.combine_embedding.combine_sparse_table,
                [(i.values(), i.offsets(), i.weights()) for i in inputs],
                [m == "mean" for m in self._modes], list(self._patch_values))
            return list(outs)
        embs = self.combine_embedding([i.values() for i in inputs])
        return [_pool(embs[k], inp.offsets(), inp.weights(), self._modes[k], self._patch_values[k])
                for k, inp in enumerate(inputs)]
