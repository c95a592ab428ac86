"""CPU engine: C++ shard per rank, gloo between ranks.

It is the plumbing path for hosts without a GPU and the executable
specification the GPU kernels are tested against.  Sparse rows are placed by
``OwnerOf`` (modulo placement, the same function the GPU shards use), dense
tables are replicated and updated from the all-reduced gradient, so N ranks
compute what one rank would on the concatenated batch.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from .._native import C
from ..utils.hashing import owner_of
from .engine import Engine, EngineConfig, TableInfo


class CpuEngine(Engine):
    def __init__(self, cfg: EngineConfig, rank: int = 0, world: int = 1, group=None) -> None:
        super().__init__(cfg, rank, world, group)
        self.shard = C.CpuShard(cfg.seed)
        self.dct_states: Dict[int, object] = {}
        self.device = torch.device("cpu")

    # ------------------------------------------------------------------ registry hooks
    def _on_init_model(self) -> None:
        self.shard.init_model(self.model_name, self.optim_type, self.optim_conf)

    def _on_register_dense(self, info: TableInfo, val: torch.Tensor) -> None:
        v = val.detach().to("cpu", torch.float32).contiguous().clone()
        if self.world > 1:
            dist.broadcast(v, src=0, group=self.group)  # one initial value for all replicas
        self.shard.create_dense_table(info.id, info.name, v)
        if self.cfg.emitter_type == C.EmitterType.kDCT:
            self.dct_states[info.id] = C.DctState()

    def _on_register_sparse(self, info: TableInfo) -> None:
        self.shard.create_sparse_table(info.id, info.name, info.dimension, info.init_type, info.init_conf)

    def _salt(self, table_id: int) -> int:
        return C.table_salt(table_id) if self.cfg.owner_salt_per_table else 0

    # ------------------------------------------------------------------ dense
    def pull_dense_table(self, table_id: int) -> torch.Tensor:
        info = self._table(table_id, "dense")
        return self.shard.pull_dense(table_id).view(*info.shape)

    def push_dense_table(self, table_id: int, grad: torch.Tensor) -> None:
        info = self._table(table_id, "dense")
        g = grad.detach().to("cpu", torch.float32).contiguous().reshape(-1)
        if g.numel() != int(torch.Size(info.shape).numel()):
            raise C.KrakenError("gradient incompatible with the dense table")
        st = self.dct_states.get(table_id)
        if st is not None:
            packed = C.cpu_dct_compress(g, self.cfg.life_span, self.cfg.eta, st)
            if packed is not None:
                idx, vals = packed
                if self.world == 1:
                    self.shard.push_dense_coo(table_id, idx, vals, self.lr)
                    return
                g = torch.zeros_like(g)
                g[idx] = vals
        if self.world > 1:
            dist.all_reduce(g, group=self.group)
        self.shard.push_dense(table_id, g, self.lr)

    # ------------------------------------------------------------------ sparse
    def _exchange(self, per_owner: List[torch.Tensor]) -> List[torch.Tensor]:
        """All-to-all of variable-length tensors (same dtype and trailing shape)."""
        send_counts = torch.tensor([int(t.shape[0]) for t in per_owner], dtype=torch.int64)
        recv_counts = torch.empty(self.world, dtype=torch.int64)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        tail = tuple(per_owner[0].shape[1:])
        width = 1
        for d in tail:
            width *= d
        send = torch.cat([t.reshape(-1) for t in per_owner]) if per_owner else torch.empty(0)
        recv = torch.empty(int(recv_counts.sum()) * width, dtype=send.dtype)
        dist.all_to_all_single(recv, send, [int(c) * width for c in recv_counts], [int(c) * width for c in send_counts],
                               group=self.group)
        out, pos = [], 0
        for c in recv_counts.tolist():
            out.append(recv[pos:pos + c * width].view(c, *tail))
            pos += c * width
        return out

    def pull_sparse_table(self, table_id: int, indices: torch.Tensor) -> torch.Tensor:
        info = self._table(table_id, "sparse")
        idx = indices.detach().to("cpu").to(torch.int64).contiguous()
        flat = idx.reshape(-1)
        uniq, inv = C.cpu_dedup(flat)
        # the push that follows a pull of the same ids (an Embedding's backward) reuses this result
        self._last_dedup = getattr(self, "_last_dedup", {})
        self._last_dedup[table_id] = (flat.clone(), uniq, inv)
        if self.world == 1:
            rows = self.shard.pull_sparse(table_id, uniq)
        else:
            owner = owner_of(self._salt(table_id), uniq, self.world)
            order = torch.argsort(owner, stable=True)
            counts = torch.bincount(owner, minlength=self.world).tolist()
            sorted_ids = uniq[order]
            per_owner = list(torch.split(sorted_ids, counts))
            asked = self._exchange(per_owner)
            answers = [self.shard.pull_sparse(table_id, a) for a in asked]
            got = self._exchange(answers)
            rows_sorted = torch.cat(got) if got else torch.empty((0, info.dimension))
            rows = torch.empty_like(rows_sorted)
            rows[order] = rows_sorted
        return rows[inv].view(*idx.shape, info.dimension)

    def push_sparse_table(self, table_id: int, indices: torch.Tensor, grad: torch.Tensor) -> None:
        info = self._table(table_id, "sparse")
        idx = indices.detach().to("cpu").to(torch.int64).contiguous().reshape(-1)
        g = grad.detach().to("cpu", torch.float32).contiguous()
        if g.numel() != idx.numel() * info.dimension:
            raise C.KrakenError("gradient shape must be indices.shape + [dimension]")
        kept = getattr(self, "_last_dedup", {}).pop(table_id, None)
        if kept is not None and kept[0].numel() == idx.numel() and torch.equal(kept[0], idx):
            uniq, inv = kept[1], kept[2]
        else:
            uniq, inv = C.cpu_dedup(idx)
        summed = C.cpu_segment_sum(g.view(-1, info.dimension), inv, uniq.numel())
        if self.world > 1:
            owner = owner_of(self._salt(table_id), uniq, self.world)
            order = torch.argsort(owner, stable=True)
            counts = torch.bincount(owner, minlength=self.world).tolist()
            ids_in = self._exchange(list(torch.split(uniq[order], counts)))
            grads_in = self._exchange(list(torch.split(summed[order], counts)))
            all_ids = torch.cat(ids_in)
            all_grads = torch.cat(grads_in)
            uniq, inv2 = C.cpu_dedup(all_ids)
            summed = C.cpu_segment_sum(all_grads, inv2, uniq.numel())
        code = self.shard.push_sparse(table_id, uniq, summed, self.lr)
        if code != 0:
            raise C.KrakenError(f"push_sparse_table: {C.error_message(code)} (code {code})")

    # ------------------------------------------------------------------ checkpoint glue
    def export_dense(self, table_id: int) -> dict:
        return self.shard.export_dense(table_id)

    def import_dense(self, table_id: int, name: str, value: dict) -> None:
        self.shard.import_dense(table_id, name, value)

    def dense_owner(self, table_id: int) -> int:
        return table_id % self.world

    def export_sparse(self, table_id: int) -> dict:
        return self.shard.export_sparse(table_id)

    def import_sparse(self, table_id: int, cols: dict) -> None:
        self.shard.import_sparse(table_id, cols["ids"], cols["vals"], cols["states"], cols["states_i"])
