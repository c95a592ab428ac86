"""NCCL-only exchange: the baseline the fused peer-memory kernels are measured against.

Same tables, same optimizer kernels, same results - but ids, rows and gradients
travel through ``torch.distributed`` collectives: an all-to-all of counts (with
the host synchronisation that sizing the next collective needs), an all-to-all
of ids, an all-to-all of rows back; dense gradients are all-reduced and every
rank updates its own full replica.  Selected with
``initialize(..., exchange="nccl")``.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .._native import C
from .sparse_shard import GpuSparseTable, SparseChannel


class NcclSparseChannel:
    def __init__(self, table: GpuSparseTable, rank: int, world: int, max_ids: int, group=None, salt: int = 0,
                 spin_limit: int = 1 << 22) -> None:
        self.table, self.rank, self.world, self.group, self.salt = table, rank, world, group, salt
        # the owner side serves the ids it receives through a single-rank channel on its own shard
        self.local = SparseChannel(table, 0, 1, max_ids * max(1, world), None, spin_limit, salt)
        self.launches = 0
        self._last = None

    def _route(self, ids: torch.Tensor):
        uniq, inv = torch.unique(ids.reshape(-1), return_inverse=True)
        owners = C.owner_of_cuda(uniq, self.salt, getattr(self, 'owner_world', self.world)).long()
        order = torch.argsort(owners, stable=True)
        send_counts = torch.bincount(owners, minlength=self.world)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        sc, rc = send_counts.tolist(), recv_counts.tolist()  # host sync: the next collective needs the sizes
        self.launches += 1
        return uniq, inv, order, sc, rc

    def _a2a(self, send: torch.Tensor, sc, rc, width: int) -> torch.Tensor:
        recv = torch.empty((sum(rc), width) if width else (sum(rc),), dtype=send.dtype, device=send.device)
        dist.all_to_all_single(recv, send.contiguous(), rc, sc, group=self.group)
        return recv

    def pull(self, ids: torch.Tensor) -> torch.Tensor:
        uniq, inv, order, sc, rc = self._route(ids)
        asked = self._a2a(uniq[order], sc, rc, 0)
        rows, _ = self.local.pull(asked)
        back = self._a2a(rows, rc, sc, self.table.dim)
        urows = torch.empty_like(back)
        urows[order] = back
        self._last = (ids.data_ptr(), ids.numel(), uniq, inv, order, sc, rc)
        return urows[inv]

    def push(self, ids: torch.Tensor, grads: torch.Tensor, lr: torch.Tensor) -> None:
        last = self._last
        if last is not None and last[0] == ids.data_ptr() and last[1] == ids.numel():
            _, _, uniq, inv, order, sc, rc = last
        else:
            uniq, inv, order, sc, rc = self._route(ids)
        dim = self.table.dim
        summed = torch.zeros((uniq.numel(), dim), dtype=torch.float32, device=grads.device)
        summed.index_add_(0, inv, grads.reshape(-1, dim).float())
        ids_in = self._a2a(uniq[order], sc, rc, 0)
        grads_in = self._a2a(summed[order], sc, rc, dim)
        self.local.push(grads_in, lr, ticket=None, ids=ids_in)
        self._last = None

    def check(self) -> None:
        self.local.check()

    def close(self) -> None:
        self.local.close()
