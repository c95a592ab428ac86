"""DeepFM on sharded sparse tables.

One dim-``dim`` table holds the second-order / deep embeddings of all fields
and one dim-1 table the first-order weights; ids are global (field offset
already added).  logit = sum_f w_f + FM2(e) + MLP([e, dense]) (the MLP's last layer carries the bias).  The
reference's example builds the same model from 39 + 39 small tables and torch
CPU ops (examples/DeepFM/model/DeepFM.py:64-140).

On the GPU engine the front end is fused around the exchange: both tables are
pulled with one shared dedup, a single kernel turns the unique rows into the
bf16 MLP input and the FM logit, and the backward kernel adds every
occurrence's gradient straight into the buffers the push sends.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .. import pytorch as kk
from .._native import C
from ..ops import counters, fm_interaction
from ..pytorch import native
from ..utils.profiler import engine_region
from .mlp import MLP


class _DeepFMFront(torch.autograd.Function):
    """Pull (one shared dedup) -> pack kernel -> (bf16 MLP input, fp32 FM logit); the backward
    kernel adds every occurrence's gradient into the push buffers.  ``first_table`` is None in
    the folded layout (first-order weight in column ``dim`` of the embedding rows)."""

    @staticmethod
    def forward(ctx, second_table, first_table, dense, ids, width, dim, in_place):
        eng = native.engine()
        id2 = second_table.table_id()
        id1 = first_table.table_id() if first_table is not None else None
        B, F = ids.shape
        # in_place: on one GPU the kernels below read the tables' rows where they are (no gather)
        rows2, inv2, t2 = eng.pull_sparse_unique(id2, ids, in_place=in_place)
        rows1 = inv1 = t1 = None
        if id1 is not None:
            rows1, inv1, t1 = eng.pull_sparse_unique(id1, ids, share_with=id2, in_place=in_place)
        x = torch.empty((B, width), dtype=torch.bfloat16, device=rows2.device)
        fm = torch.empty(B, dtype=torch.float32, device=rows2.device)
        ssum = torch.empty((B, dim), dtype=torch.float32, device=rows2.device)  # sum_f e_f, reused by the backward
        dense = dense.to(rows2.device, torch.float32).contiguous()
        counters.add()
        with engine_region("pack_fwd"):
            C.deepfm_pack_forward(rows2, inv2, rows1, inv1, dense, B, F, dim, x, fm, t2.slots,
                                  t1.slots if t1 is not None else None, ssum)
        ctx.state = (eng, id1, id2, rows2, inv2, inv1, t1, t2, B, F, dim, ssum)
        return x, fm

    @staticmethod
    def backward(ctx, dx, dfm):
        eng, id1, id2, rows2, inv2, inv1, t1, t2, B, F, dim, ssum = ctx.state
        if dfm is None:
            dfm = torch.zeros(B, dtype=torch.float32, device=rows2.device)
        counters.add()
        with engine_region("pack_bwd"):
            C.deepfm_pack_backward(rows2, inv2, inv1, dx.contiguous() if dx is not None else None,
                                   dfm.float().contiguous(), B, F, dim, eng.grad_accumulator(id2),
                                   eng.grad_accumulator(id1) if id1 is not None else None, t2.slots, ssum)
        if id1 is not None:
            eng.push_sparse_accumulated(id1, t1)
        eng.push_sparse_accumulated(id2, t2)
        return None, None, None, None, None, None, None


class DeepFM(torch.nn.Module):
    def __init__(self, num_fields: int = 26, num_dense: int = 13, dim: int = 16,
                 hidden: Sequence[int] = (400, 400, 400), init_std: float = 0.01, name: str = "deepfm",
                 fused: bool = True, fold_first_order: bool = False, in_place_rows: Optional[bool] = None):
        """fold_first_order: keep each id's first-order weight in the same table row as its
        embedding (row = dim embedding floats + 1 weight, padded to a multiple of 4), so a step
        needs one sparse exchange instead of two.  Only the fused GPU path reads that layout.
        in_place_rows: on a single GPU read the table rows where they are instead of gathering the
        unique rows first (one launch fewer; pays off for small batches, costs L2 locality for large
        ones).  None = decide per call from the number of ids (measured crossover: about 0.5 M)."""
        super().__init__()
        self.num_fields, self.num_dense, self.dim = num_fields, num_dense, dim
        self.fold = bool(fold_first_order)
        if self.fold:
            self.row_dim = (dim + 1 + 3) // 4 * 4
            self.first_order = None
            self.second_order = kk.Embedding(self.row_dim, initializer=kk.NormalInitializer(0.0, init_std),
                                             name=f"{name}.embedding_and_first_order")
        else:
            self.row_dim = dim
            self.first_order = kk.Embedding(1, initializer=kk.ConstantInitializer(0.0), name=f"{name}.first_order")
            self.second_order = kk.Embedding(dim, initializer=kk.NormalInitializer(0.0, init_std),
                                             name=f"{name}.second_order")
        width = num_fields * dim + num_dense
        self.mlp_in = (width + 7) // 8 * 8  # padded: the tensor-core path wants pitches in multiples of 8
        self.pad = self.mlp_in - width
        self.mlp = MLP(self.mlp_in, list(hidden) + [1])
        self.fused = fused
        self.in_place_rows = in_place_rows

    def _fused_ok(self, ids: torch.Tensor) -> bool:
        chunks = self.dim // 4
        return (self.fused and self.dim % 4 == 0 and chunks & (chunks - 1) == 0 and self.dim <= 128 and ids.dim() == 2 and native.is_initialized()
                and hasattr(native.engine(), "pull_sparse_unique") and not getattr(native.engine(), "nccl", False)
                and self.mlp.use_tensor_cores)

    def forward(self, dense: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
        if self._fused_ok(ids):
            first = self.first_order.sparse_table if self.first_order is not None else None
            prepared = self.mlp.prepare()  # weight casts run beside the sparse pull
            x, fm = _DeepFMFront.apply(self.second_order.sparse_table, first, dense, ids, self.mlp_in, self.dim,
                                       self.in_place_rows if self.in_place_rows is not None
                                       else ids.numel() <= (1 << 19))
            return self.mlp(x, input_grad_cols=self.num_fields * self.dim, addend=fm, prepared=prepared).squeeze(-1)
        if self.fold:
            rows = self.second_order(ids)                    # [B, F, row_dim]
            e, w = rows[..., :self.dim], rows[..., self.dim:self.dim + 1]
        else:
            w = self.first_order(ids)   # [B, F, 1]
            e = self.second_order(ids)  # [B, F, dim]
        dense = dense.to(e.device)
        parts = [e.flatten(1), dense]
        if self.pad:
            parts.append(torch.zeros(dense.shape[0], self.pad, dtype=e.dtype, device=e.device))
        deep = self.mlp(torch.cat(parts, dim=1)).squeeze(-1)
        return w.sum(dim=(1, 2)) + fm_interaction(e.contiguous()) + deep
