"""GPU engine: every rank is a worker and a shard on its own B200.

Sparse tables are ``GpuSparseTable`` shards exchanged through ``SparseChannel``
(fused pull / push kernels over peer memory); dense tables live in one
``DenseBucket`` whose fused step replaces push + server update + pull.  No call
here synchronises the host: errors are collected from device status words by
``check()`` / ``end_step()``.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from .._native import C
from ..parallel.dense_bucket import BucketSet
from ..parallel.nccl_baseline import NcclSparseChannel
from ..parallel.sparse_shard import GpuSparseTable, GroupChannel, SparseChannel, Ticket
from ..utils import profiler as _profiler
from .engine import Engine, EngineConfig, TableInfo


class GpuEngine(Engine):
    def __init__(self, cfg: EngineConfig, rank: int = 0, world: int = 1, group=None,
                 device: Optional[torch.device] = None) -> None:
        super().__init__(cfg, rank, world, group)
        if not torch.cuda.is_available():
            raise RuntimeError("the GPU engine needs a CUDA device")
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        torch.cuda.set_device(self.device)
        self.lr_dev = torch.zeros(1, dtype=torch.float32, device=self.device)
        self._lr_host = torch.zeros(1, dtype=torch.float32).pin_memory()
        self.sparse: Dict[int, GpuSparseTable] = {}
        self.channels: Dict[int, SparseChannel] = {}
        self.tickets: Dict[int, Tuple[Ticket, int, int, int]] = {}
        self.group_channels: Dict[Tuple[int, ...], GroupChannel] = {}
        self.group_tickets: Dict[Tuple[int, ...], tuple] = {}
        self.owner_world = world   # sparse rows live on ranks 0 .. owner_world - 1; reshard() changes it
        self.dense_init: Dict[int, torch.Tensor] = {}
        self.bucket: Optional[BucketSet] = None
        self._comm_stream: Optional[torch.cuda.Stream] = None
        self._param_table: Dict[int, int] = {}     # id(parameter) -> dense table id (bound parameters)
        self._bucket_ready: Dict[int, set] = {}     # bucket -> tables whose gradient is complete this step
        self._dense_pending = False
        self._pushed: set = set()
        self._bound = False
        self._steps = 0
        self.profiler = _profiler.from_env(rank)
        self._nvtx = os.environ.get("KRAKEN_NVTX", "") == "1"
        self.nccl = cfg.exchange == "nccl" and world > 1
        self.nccl_channels: Dict[int, NcclSparseChannel] = {}
        from ..ops import mlp as fused_mlp
        fused_mlp.set_deferred_join(bool(cfg.overlap_dense_step) and not self.nccl)

    # ------------------------------------------------------------------ registry hooks
    def _on_update_lr(self) -> None:
        if float(self._lr_host[0]) != self.lr or self._steps == 0:
            self._lr_host[0] = self.lr
            self.lr_dev.copy_(self._lr_host, non_blocking=True)

    def _on_register_dense(self, info: TableInfo, val: torch.Tensor) -> None:
        v = val.detach().to(self.device, torch.float32).contiguous().clone()
        if self.world > 1:
            dist.broadcast(v, src=0, group=self.group)
        self.dense_init[info.id] = v
        if self.bucket is not None:
            self._rebuild_bucket()

    def _on_register_sparse(self, info: TableInfo) -> None:
        self.sparse[info.id] = GpuSparseTable(info.id, info.name, info.dimension, info.init_type, info.init_conf,
                                              self.optim_type, self.optim_conf, self.cfg.seed,
                                              self.cfg.table_capacity, self.world, self.device)

    def _salt(self, table_id: int) -> int:
        return C.table_salt(table_id) if self.cfg.owner_salt_per_table else 0

    # ------------------------------------------------------------------ dense
    def _dense_ids(self) -> List[int]:
        return [tid for tid, t in self.tables.items() if t.kind == "dense"]

    def _build_bucket(self) -> None:
        ids = self._dense_ids()
        tables = [(tid, int(self.dense_init[tid].numel())) for tid in ids]
        b_rank, b_world = (0, 1) if self.nccl else (self.rank, self.world)
        self.bucket = BucketSet(tables, self.optim_type, self.optim_conf, b_rank, b_world, self.device,
                                self.group, dct=self.cfg.emitter_type == C.EmitterType.kDCT,
                                life_span=self.cfg.life_span, eta=self.cfg.eta, spin_limit=self.cfg.spin_limit,
                                bucket_elems=self.cfg.dense_bucket_elems)
        for tid in ids:
            self.bucket.param_view(tid, self.tables[tid].shape).copy_(self.dense_init[tid].view(*self.tables[tid].shape))
        if self.world > 1:
            torch.cuda.synchronize()
            dist.barrier(group=self.group)

    def _rebuild_bucket(self) -> None:
        old = self.bucket
        for tid in old.table_ids:
            self.dense_init[tid] = old.param_view(tid, self.tables[tid].shape).detach().clone().reshape(-1)
        # optimizer state of the old bucket is dropped: tables are registered before training starts
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier(group=self.group)
        old.close()
        self.bucket = None
        self._build_bucket()

    def _ensure_bucket(self) -> DenseBucket:
        if self.bucket is None:
            self._build_bucket()
        return self.bucket

    def pull_dense_table(self, table_id: int) -> torch.Tensor:
        info = self._table(table_id, "dense")
        b = self._ensure_bucket()
        self._flush_dense()
        return b.param_view(table_id, info.shape)

    def combine_pull_dense_table(self, table_ids: Sequence[int]) -> List[torch.Tensor]:
        if not table_ids:
            return []
        b = self._ensure_bucket()
        self._flush_dense()
        return [b.param_view(t, self._table(t, "dense").shape) for t in table_ids]

    def push_dense_table(self, table_id: int, grad: torch.Tensor) -> None:
        info = self._table(table_id, "dense")
        b = self._ensure_bucket()
        view = b.grad_view(table_id, info.shape)
        if grad.data_ptr() != view.data_ptr():
            view.add_(grad.detach().to(self.device, torch.float32).view(*info.shape))
        self._pushed.add(table_id)
        self._dense_pending = True

    def bind_dense_params(self, pairs: Sequence[Tuple[int, torch.nn.Parameter]]) -> None:
        """Makes each parameter alias the bucket: ``.data`` is the parameter view and
        ``.grad`` the gradient view, so backward accumulates into the exchange buffer."""
        b = self._ensure_bucket()
        from ..ops import mlp as fused_mlp
        for tid, p in pairs:
            shape = self._table(tid, "dense").shape
            p.data = b.param_view(tid, shape)
            p.grad = b.grad_view(tid, shape)
            self._param_table[id(p)] = tid
            if self.cfg.overlap_dense_step and hasattr(p, "register_post_accumulate_grad_hook"):
                # gradients that autograd accumulates (layers outside the fused MLP) report through this hook;
                # the fused MLP writes its gradients from its own kernels and reports them itself
                p.register_post_accumulate_grad_hook(lambda param: self.dense_grad_ready(param))
        if self.cfg.overlap_dense_step and not self.nccl:
            fused_mlp.set_grad_ready_callback(self.dense_grad_ready)
        self._bound = True

    def dense_grad_ready(self, param, stream: Optional[torch.cuda.Stream] = None) -> None:
        """The gradient of a bound dense parameter is complete for this step (all kernels that write it are
        enqueued on ``stream``, default: the current one).  When that completes a bucket, its fused step
        (reduce-scatter + optimizer + all-gather) is launched at once on the communication stream, behind an
        event on ``stream``, so it overlaps the rest of the backward pass.  Only with ``overlap_dense_step``;
        every rank sees the same parameters complete in the same order, so the launches stay collective."""
        tid = self._param_table.get(id(param))
        b = self.bucket
        if tid is None or b is None or self.nccl or not self.cfg.overlap_dense_step:
            return
        k = b.bucket_of[tid]
        ready = self._bucket_ready.setdefault(k, set())
        ready.add(tid)
        if len(ready) < len(b.buckets[k].table_ids) or len(b.buckets) == 1:
            return  # a single bucket is stepped by dense_step(), on the stream the last gradients were written on
        src = stream or torch.cuda.current_stream(self.device)
        if self._comm_stream is None:
            self._comm_stream = torch.cuda.Stream(device=self.device)
        ev = torch.cuda.Event()
        ev.record(src)
        self._comm_stream.wait_event(ev)
        b.buckets[k].set_active([True] * len(b.buckets[k].table_ids))
        with self._region("dense_step"), torch.cuda.stream(self._comm_stream):
            b.step_bucket(k, self.lr_dev)
        self._comm_used = True

    def dense_step(self) -> None:
        """One fused optimizer step over every dense table (bound-parameter path)."""
        b = self._ensure_bucket()
        b.set_active([True] * len(b.table_ids))
        with self._region("dense_step"):
            if self.nccl:
                for g in b.grads():
                    dist.all_reduce(g, group=self.group)
            from ..ops import mlp as fused_mlp
            side = fused_mlp.take_pending_side_stream(self.device) if not self.nccl else None
            main = torch.cuda.current_stream(self.device)
            if side is not None:
                # the MLP backward left its weight gradients on this stream: step (what is left) there, then join
                with torch.cuda.stream(side):
                    b.step(self.lr_dev)
                main.wait_stream(side)
            else:
                b.step(self.lr_dev)
            if getattr(self, "_comm_used", False):
                main.wait_stream(self._comm_stream)  # buckets that were stepped during the backward pass
                self._comm_used = False
        self._bucket_ready.clear()
        self._dense_pending = False
        self._pushed.clear()

    def _region(self, name: str):
        """Phase bracket: CUDA-event timing when KRAKEN_PROFILE is set, an NVTX range when KRAKEN_NVTX=1
        (for timeline tools), nothing otherwise."""
        import contextlib
        if self.profiler is not None:
            return self.profiler.region(name)
        if self._nvtx:
            return torch.cuda.nvtx.range(f"kraken.{name}")
        return contextlib.nullcontext()

    def metrics(self) -> dict:
        """Counters of the shards (synchronises): rows and load factor per sparse table and, where
        a table has been used, its latest exchange (occurrences, unique ids, bytes over NVLink)."""
        out = {}
        for tid, t in self.sparse.items():
            rows = t.num_rows()
            rec = {"rows": rows, "capacity": t.capacity, "load_factor": rows / t.capacity}
            ch = self.channels.get(tid)
            if ch is not None and hasattr(ch, "last_exchange"):
                rec["last_exchange"] = ch.last_exchange()
            out[self.tables[tid].name] = rec
        return out

    def _flush_dense(self) -> None:
        if not self._dense_pending:
            return
        b = self.bucket
        b.set_active([tid in self._pushed for tid in b.table_ids])
        if self.nccl:
            for g in b.grads():
                dist.all_reduce(g, group=self.group)
        b.step(self.lr_dev)
        self._dense_pending = False
        self._pushed.clear()

    # ------------------------------------------------------------------ sparse
    def _channel(self, table_id: int, n: int) -> SparseChannel:
        ch = self.channels.get(table_id)
        if ch is not None:
            return ch
        cap = self.cfg.max_ids_per_call
        if cap <= 0:
            cap = max(1024, 2 * n)
            if self.world > 1:
                t = torch.tensor([cap], dtype=torch.int64, device=self.device)
                dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
                cap = int(t.item())
        ch = SparseChannel(self.sparse[table_id], self.rank, self.world, cap, self.group, self.cfg.spin_limit,
                           self._salt(table_id), max_unique=self.cfg.max_unique_per_call,
                           max_per_owner=self.cfg.max_per_owner_per_call)
        ch.owner_world = self.owner_world
        self.channels[table_id] = ch
        return ch

    def _prep_ids(self, indices: torch.Tensor) -> torch.Tensor:
        idx = indices.detach()
        if idx.device != self.device or idx.dtype != torch.int64:
            idx = idx.to(self.device, torch.int64, non_blocking=True)
        return idx.contiguous()

    @staticmethod
    def _sig(indices: torch.Tensor) -> Tuple[int, int, int]:
        return (indices.data_ptr(), indices.numel(), indices._version)

    def _remember(self, table_id: int, ticket, indices: torch.Tensor) -> None:
        """Keeps the pull's ticket for the push that follows.  The indices tensor itself is kept alive with
        it: a ticket is matched by address + version, and memory of a freed tensor could be handed to a
        DIFFERENT id tensor of the same size, whose push would then update the rows of the earlier pull."""
        self.tickets[table_id] = (ticket, indices, *self._sig(indices))

    def _recall(self, table_id: int, indices: torch.Tensor):
        saved = self.tickets.pop(table_id, None)
        if saved is None or saved[2:] != self._sig(indices):
            return None
        return saved[0]

    def _nccl_channel(self, table_id: int, n: int) -> NcclSparseChannel:
        ch = self.nccl_channels.get(table_id)
        if ch is None:
            cap = self.cfg.max_ids_per_call or max(1024, 2 * n)
            t = torch.tensor([cap], dtype=torch.int64, device=self.device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
            ch = NcclSparseChannel(self.sparse[table_id], self.rank, self.world, int(t.item()), self.group,
                                   self._salt(table_id), self.cfg.spin_limit)
            ch.owner_world = self.owner_world
            self.nccl_channels[table_id] = ch
        return ch

    def pull_sparse_table(self, table_id: int, indices: torch.Tensor) -> torch.Tensor:
        info = self._table(table_id, "sparse")
        idx = self._prep_ids(indices)
        if self.nccl:
            self._ensure_room(table_id, idx.numel())
            rows = self._nccl_channel(table_id, idx.numel()).pull(idx)
            self._nccl_ids = {**getattr(self, "_nccl_ids", {}), table_id: (indices, *self._sig(indices), idx)}
            return rows.view(*indices.shape, info.dimension)
        ch = self._channel(table_id, idx.numel())
        if self.cfg.long_id_streams:
            rounds = self._rounds(idx.numel(), ch.cap)
            if rounds > 1:
                return self._pull_in_rounds(table_id, ch, idx, rounds).view(*indices.shape, info.dimension)
        self._ensure_room(table_id, idx.numel())
        with self._region("pull"):
            rows, ticket = ch.pull(idx)
        self._remember(table_id, ticket, indices)
        return rows.view(*indices.shape, info.dimension)

    # ------------------------------------------------------------------ id streams longer than the buffers
    def _rounds(self, n: int, cap: int) -> int:
        """How many exchanges of at most ``cap`` ids a call of ``n`` ids needs - the maximum over the ranks,
        because every exchange is collective: a rank with fewer ids joins the later rounds with none."""
        r = max(1, -(-int(n) // int(cap)))
        if self.world > 1:
            t = torch.tensor([r], dtype=torch.int64, device=self.device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
            r = int(t.item())
        return r

    def _pull_in_rounds(self, table_id: int, ch: SparseChannel, idx: torch.Tensor, rounds: int) -> torch.Tensor:
        """The chunked exchange for long id streams: round k looks up ids [k * cap, (k + 1) * cap) through the
        same buffers (the reference's emitter has no size limit per request, kraken/worker/emitter.cc:123-183).
        No ticket is kept: the push that follows deduplicates its own rounds."""
        flat = idx.reshape(-1)
        out = torch.empty((flat.numel(), ch.table.dim), dtype=torch.float32, device=self.device)
        self.tickets.pop(table_id, None)
        with self._region("pull"):
            for k in range(rounds):
                part = flat[k * ch.cap:(k + 1) * ch.cap]
                self._ensure_room(table_id, part.numel())
                ch.pull(part, out=out[k * ch.cap:k * ch.cap + part.numel()])
        return out

    def _push_in_rounds(self, ch: SparseChannel, idx: torch.Tensor, g: torch.Tensor, rounds: int) -> None:
        """Push of a long id stream.  An id that occurs in several rounds is updated once per round it occurs
        in (the reference applies one update per request too); within a round duplicates are summed first."""
        flat, g2 = idx.reshape(-1), g.reshape(-1, ch.table.dim)
        with self._region("push"):
            for k in range(rounds):
                a, b = k * ch.cap, min((k + 1) * ch.cap, flat.numel())
                a = min(a, b)
                ch.push(g2[a:b], self.lr_dev, ticket=None, ids=flat[a:b])

    # ------------------------------------------------------------------ several tables, one exchange
    def _group_channel(self, tids: Tuple[int, ...], n_total: int) -> GroupChannel:
        ch = self.group_channels.get(tids)
        if ch is not None:
            return ch
        cap = max(1024, 2 * n_total)
        if self.world > 1:
            t = torch.tensor([cap], dtype=torch.int64, device=self.device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
            cap = int(t.item())
        ch = GroupChannel([self.sparse[t] for t in tids], self.rank, self.world, cap, self.group, self.cfg.spin_limit,
                          salts=[self._salt(t) for t in tids])
        ch.owner_world = self.owner_world
        self.group_channels[tids] = ch
        return ch

    def _dim_classes(self, table_ids: Sequence[int]):
        """Positions of ``table_ids`` grouped by row width, in first-appearance order; None when a table is
        named twice (each call then goes through its own exchange)."""
        if len(set(table_ids)) != len(table_ids):
            return None
        classes: Dict[int, List[int]] = {}
        for pos, t in enumerate(table_ids):
            classes.setdefault(self._table(t, "sparse").dimension, []).append(pos)
        return classes

    def combine_pull_sparse_table(self, table_ids: Sequence[int], indices: Sequence[torch.Tensor]) -> List[torch.Tensor]:
        """All tables of one row width share ONE exchange (dedup keyed by (table, id), one dispatch, one
        gather), as the reference's combined request does in one round per server
        (kraken/worker/emitter.cc:185-278); tables of different widths form one group per width."""
        if len(table_ids) != len(indices):
            raise C.KrakenError("table_ids and indices differ in length")
        classes = None if self.nccl else self._dim_classes(table_ids)
        if classes is None or all(len(p) == 1 for p in classes.values()):
            return super().combine_pull_sparse_table(table_ids, indices)
        out: List[Optional[torch.Tensor]] = [None] * len(table_ids)
        for dim, pos in classes.items():
            if len(pos) == 1:
                out[pos[0]] = self.pull_sparse_table(table_ids[pos[0]], indices[pos[0]])
                continue
            tids = tuple(int(table_ids[p]) for p in pos)
            flat = [self._prep_ids(indices[p]).reshape(-1) for p in pos]
            counts = [int(f.numel()) for f in flat]
            ch = self._group_channel(tids, sum(counts))
            for t, c in zip(tids, counts):
                self._ensure_room(t, c)
            with self._region("pull"):
                rows, ticket = ch.pull(torch.cat(flat), counts)
            self.group_tickets[tids] = (ticket, [indices[p] for p in pos], [self._sig(indices[p]) for p in pos])
            for p, part in zip(pos, rows.split(counts)):
                out[p] = part.view(*indices[p].shape, dim)
        return out

    def combine_push_sparse_table(self, table_ids: Sequence[int], indices: Sequence[torch.Tensor],
                                  grads: Sequence[torch.Tensor]) -> None:
        if not (len(table_ids) == len(indices) == len(grads)):
            raise C.KrakenError("table_ids, indices and grads differ in length")
        classes = None if self.nccl else self._dim_classes(table_ids)
        if classes is None or all(len(p) == 1 for p in classes.values()):
            return super().combine_push_sparse_table(table_ids, indices, grads)
        for dim, pos in reversed(list(classes.items())):
            if len(pos) == 1:
                self.push_sparse_table(table_ids[pos[0]], indices[pos[0]], grads[pos[0]])
                continue
            tids = tuple(int(table_ids[p]) for p in pos)
            grads = list(grads)
            for p in pos:
                if grads[p] is None:  # an output autograd never used
                    grads[p] = torch.zeros((int(indices[p].numel()), dim), dtype=torch.float32, device=self.device)
                if grads[p].numel() != indices[p].numel() * dim:
                    raise C.KrakenError("gradient shape must be indices.shape + [dimension]")
            saved = self.group_tickets.pop(tids, None)
            ticket = saved[0] if saved is not None and saved[2] == [self._sig(indices[p]) for p in pos] else None
            g = torch.cat([grads[p].detach().to(self.device, torch.float32).reshape(-1, dim) for p in pos])
            ch = self._group_channel(tids, sum(int(indices[p].numel()) for p in pos))
            with self._region("push"):
                if ticket is not None:
                    ch.push(g, self.lr_dev, ticket=ticket)
                else:
                    flat = [self._prep_ids(indices[p]).reshape(-1) for p in pos]
                    ch.push(g, self.lr_dev, ids_cat=torch.cat(flat), counts=[int(f.numel()) for f in flat])

    def combine_pull_sparse_pooled(self, table_ids: Sequence[int], inputs, means: Sequence[bool],
                                   patch_values: Sequence[float]):
        """EmbeddingBag lookups of several tables.  ``inputs[k]`` = (values, offsets, weights or None) of table
        k.  Tables of equal row width and patch value go through ONE combined exchange whose pooled gather
        handles per-bag sum / mean; the others take the single-table fused path.  Returns (pooled outputs in
        table order, handles for ``combine_push_sparse_pooled``)."""
        n_tab = len(table_ids)
        if not (n_tab == len(inputs) == len(means) == len(patch_values)):
            raise C.KrakenError("table_ids, inputs, means and patch_values differ in length")
        outs: List[Optional[torch.Tensor]] = [None] * n_tab
        handles = []
        classes: Dict[Tuple[int, float], List[int]] = {}
        if len(set(table_ids)) == n_tab:
            for pos, t in enumerate(table_ids):
                classes.setdefault((self._table(t, "sparse").dimension, float(patch_values[pos])), []).append(pos)
        else:
            classes = {(-pos - 1, 0.0): [pos] for pos in range(n_tab)}  # a table named twice: one exchange each
        for (dim, patch), pos in classes.items():
            if len(pos) == 1:
                p = pos[0]
                v, o, w = inputs[p]
                out, ticket = self.pull_sparse_pooled(table_ids[p], v, o, weights=w, mean=bool(means[p]),
                                                      patch_value=float(patch_values[p]))
                outs[p] = out
                handles.append(("single", int(table_ids[p]), ticket, v, [p]))
                continue
            tids = tuple(int(table_ids[p]) for p in pos)
            vals = [self._prep_ids(inputs[p][0]).reshape(-1) for p in pos]
            counts = [int(v.numel()) for v in vals]
            offs, bags, base = [], [], 0
            for k, p in enumerate(pos):
                o = inputs[p][1].detach().to(self.device, torch.int64)
                offs.append(o + base if k == 0 else o[1:] + base)
                bags.append(int(o.numel()) - 1)
                base += counts[k]
            weights = None
            if any(inputs[p][2] is not None for p in pos):
                weights = torch.cat([inputs[p][2].detach().to(self.device, torch.float32).reshape(-1)
                                     if inputs[p][2] is not None else torch.ones(counts[k], device=self.device)
                                     for k, p in enumerate(pos)])
            bag_mean = torch.cat([torch.full((bags[k],), 1 if means[p] else 0, dtype=torch.uint8, device=self.device)
                                  for k, p in enumerate(pos)])
            ch = self._group_channel(tids, sum(counts))
            for t, c in zip(tids, counts):
                self._ensure_room(t, c)
            with self._region("pull"):
                rows, ticket = ch.pull(torch.cat(vals), counts, bag_offsets=torch.cat(offs).contiguous(),
                                       weights=weights, bag_mean=bag_mean, patch_value=patch)
            for p, part in zip(pos, rows.split(bags)):
                outs[p] = part
            handles.append(("group", tids, ticket, (vals, counts, bags), list(pos)))
        return outs, handles

    def combine_push_sparse_pooled(self, handles, grads: Sequence[Optional[torch.Tensor]]) -> None:
        for kind, key, ticket, ids, pos in reversed(handles):
            if kind == "single":
                g = grads[pos[0]]
                if g is None:
                    continue
                self.push_sparse_pooled(key, ticket, g.contiguous(), ids)
                continue
            ch = self.group_channels[key]
            dim = ch.dim
            vals, counts, bags = ids
            parts = []
            for k, p in enumerate(pos):
                g = grads[p]
                if g is None:  # an output autograd never used
                    g = torch.zeros((bags[k], dim), dtype=torch.float32, device=self.device)
                elif g.numel() != bags[k] * dim:
                    raise C.KrakenError("gradient rows do not match the bags of the combined lookup")
                parts.append(g.detach().to(self.device, torch.float32).reshape(-1, dim))
            g_cat = torch.cat(parts)
            with self._region("push"):
                if ticket.channel is ch and ticket.serial == ch.serial:
                    ch.push(g_cat, self.lr_dev, ticket=ticket)
                else:
                    # another lookup used the channel in between: resolve the ids again, pool shape from the ticket
                    n = ch._lookup_phase(torch.cat(vals), counts, insert=False)
                    t2 = Ticket(ch, ch.serial, n, ticket.bag_offsets, ticket.weights, False, ticket.bag_mean)
                    ch.push(g_cat, self.lr_dev, ticket=t2)

    def pull_sparse_pooled(self, table_id: int, values: torch.Tensor, offsets: torch.Tensor,
                           weights: Optional[torch.Tensor] = None, mean: bool = False,
                           bag_mean: Optional[torch.Tensor] = None, patch_value: float = 0.0):
        """EmbeddingBag in one fused pull: returns (pooled [k, dim], ticket)."""
        self._table(table_id, "sparse")
        idx = self._prep_ids(values)
        off = offsets.detach().to(self.device, torch.int64).contiguous()
        w = weights.detach().to(self.device, torch.float32).contiguous() if weights is not None else None
        bm = bag_mean.detach().to(self.device, torch.uint8).contiguous() if bag_mean is not None else None
        ch = self._channel(table_id, idx.numel())
        self._ensure_room(table_id, idx.numel())
        return ch.pull(idx, bag_offsets=off, weights=w, mean=mean, bag_mean=bm, patch_value=patch_value)

    def push_sparse_pooled(self, table_id: int, ticket: Ticket, grads: torch.Tensor,
                           values: Optional[torch.Tensor] = None) -> None:
        ch = self.channels[table_id]
        ids = self._prep_ids(values) if values is not None else None
        ch.push(grads, self.lr_dev, ticket=ticket, ids=ids, bag_offsets=ticket.bag_offsets, weights=ticket.weights,
                mean=ticket.mean, bag_mean=ticket.bag_mean)

    def pull_sparse_unique(self, table_id: int, indices: torch.Tensor, share_with: Optional[int] = None,
                           in_place: bool = False):
        """Pull for fused consumers: (unique rows buffer, occurrence -> unique map, ticket).
        ``share_with`` names a table whose channel has just pulled the same ids: its
        dedup result is reused.  ``in_place``: on a single GPU return the table's value slab and
        the slot of every unique entry (``ticket.slots``) instead of copying the rows."""
        self._table(table_id, "sparse")
        idx = self._prep_ids(indices)
        ch = self._channel(table_id, idx.numel())
        share = self.channels.get(share_with) if share_with is not None else None
        self._ensure_room(table_id, idx.numel())
        with self._region("pull"):
            return ch.pull_unique(idx, share_from=share, in_place=in_place)

    def grad_accumulator(self, table_id: int) -> torch.Tensor:
        """Per-unique-id gradient buffer [cap, dim] of the table's channel (zero between steps)."""
        return self.channels[table_id].ugrad

    def push_sparse_accumulated(self, table_id: int, ticket: Ticket) -> None:
        with self._region("push"):
            self.channels[table_id].push_accumulated(self.lr_dev, ticket)

    def push_sparse_table(self, table_id: int, indices: torch.Tensor, grad: torch.Tensor) -> None:
        info = self._table(table_id, "sparse")
        if grad.numel() != indices.numel() * info.dimension:
            raise C.KrakenError("gradient shape must be indices.shape + [dimension]")
        if self.nccl:
            kept = getattr(self, "_nccl_ids", {}).pop(table_id, None)
            idx = kept[4] if kept is not None and kept[1:4] == self._sig(indices) else self._prep_ids(indices)
            self._nccl_channel(table_id, idx.numel()).push(idx, grad.detach().to(self.device), self.lr_dev)
            return
        ticket = self._recall(table_id, indices)
        idx = None if ticket is not None else self._prep_ids(indices)
        ch = self._channel(table_id, indices.numel())
        g = grad.detach()
        if g.device != self.device:
            g = g.to(self.device)
        if self.cfg.long_id_streams:
            rounds = self._rounds(indices.numel(), ch.cap)
            if rounds > 1:
                return self._push_in_rounds(ch, self._prep_ids(indices), g.to(torch.float32), rounds)
        with self._region("push"):
            ch.push(g, self.lr_dev, ticket=ticket, ids=idx)

    # ------------------------------------------------------------------ live reshard
    def reshard(self, owner_world: int) -> int:
        """Changes, inside the running job, how many of the ranks hold sparse rows: afterwards row ``id`` of a
        table lives on rank ``OwnerOf(salt, id, owner_world)`` (ranks >= owner_world hold none and act as workers
        only).  Collective, between steps.  Every rank compacts the rows it no longer owns on the device
        (``table_export`` with the owner filter), sends each with its optimizer state and step count to the new
        owner (one all-to-all per table), rebuilds its own table from the rows it keeps and inserts what it
        receives - the scale-out / scale-in of kraken/ps/ps.cc:125-372 (TransferTo, CleanTables) without files.
        Returns how many rows this rank sent away."""
        owner_world = int(owner_world)
        if not 1 <= owner_world <= self.world:
            raise C.KrakenError(f"owner_world must be between 1 and {self.world}")
        if owner_world == self.owner_world:
            return 0
        torch.cuda.synchronize(self.device)
        sent = 0
        dev = self.device
        for tid, t in sorted(self.sparse.items()):
            salt = self._salt(tid)
            away = t.export(filter_mode=2, salt=salt, world=owner_world, rank=self.rank)   # rows another rank will own
            keep = t.export(filter_mode=1, salt=salt, world=owner_world, rank=self.rank)
            n = int(away["ids"].numel())
            sent += n
            skeys = sorted(int(k) for k in away["states"])
            has_steps = 0 in away["states_i"]
            owners = (C.owner_of_cuda(away["ids"], salt, owner_world).long() if n
                      else torch.empty(0, dtype=torch.long, device=dev))
            order = torch.argsort(owners, stable=True)
            send = torch.bincount(owners, minlength=self.world)
            recv = torch.empty_like(send)
            if self.world > 1:
                dist.all_to_all_single(recv, send, group=self.group)
            else:
                recv.copy_(send)
            sc, rc = send.tolist(), recv.tolist()

            def a2a(x: torch.Tensor, width: int) -> torch.Tensor:
                out = torch.empty((sum(rc), width) if width else (sum(rc),), dtype=x.dtype, device=dev)
                if self.world > 1:
                    dist.all_to_all_single(out, x[order].contiguous(), rc, sc, group=self.group)
                else:
                    out.copy_(x[order])
                return out

            in_ids = a2a(away["ids"], 0)
            in_vals = a2a(away["vals"], t.dim)
            in_states = {k: a2a(away["states"][k], t.dim) for k in skeys}
            in_steps = {0: a2a(away["states_i"][0], 0)} if has_steps else {}
            C.table_clear(t.host())
            t.val.zero_()
            for k, slab in enumerate(t.slabs):
                if slab is not None:
                    slab.fill_(t.optim_info["initial_accumulator_value"] if (t.optim_info["type"] == 0 and k == 0) else 0.0)
            if t.steps is not None:
                t.steps.zero_()
            t.rows_hi = 0
            t.import_rows(keep["ids"], keep["vals"], keep["states"], keep["states_i"])
            t.import_rows(in_ids, in_vals, in_states, in_steps)
        self.owner_world = owner_world
        for ch in list(self.channels.values()) + list(self.group_channels.values()) + list(self.nccl_channels.values()):
            ch.owner_world = owner_world
        self.tickets.clear()         # slots resolved before the move are stale
        self.group_tickets.clear()
        for ch in self.channels.values():
            ch.serial += 1
        for ch in self.group_channels.values():
            ch.serial += 1
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(group=self.group)
        return sent

    # ------------------------------------------------------------------ housekeeping
    def end_step(self) -> bool:
        """Between steps: grows tables whose load factor passed the limit and surfaces errors that
        kernels recorded (table full, inbox overflow, a wait that timed out, push to an unknown id) as
        ``KrakenError`` - the reference answers every RPC with an error code, here the codes are
        collected from device memory without stalling the step: the words are copied to pinned memory
        every ``status_poll_interval`` steps and examined once that copy has landed.  Returns True when
        a table was reallocated (a captured CUDA graph of the step is stale then)."""
        if torch.cuda.is_current_stream_capturing():
            return False  # growth checks use events and may reallocate: not inside a graph capture
        self._steps += 1
        if self.profiler is not None:
            self.profiler.end_step()
        grew = False
        for t in self.sparse.values():
            grew = t.poll_growth() or grew
        self._poll_status()
        return grew

    def _status_words(self):
        """(label, 1-element int32 device tensor) of every status word kernels of this engine write."""
        out = []
        for tid, ch in self.channels.items():
            out.append((f"exchange of table {self.tables[tid].name!r}", ch.ctrl[4:5]))
        for tid, ch in self.nccl_channels.items():
            out.append((f"exchange of table {self.tables[tid].name!r}", ch.local.ctrl[4:5]))
        for tids, ch in self.group_channels.items():
            out.append((f"combined exchange of tables {list(tids)}", ch.ctrl[4:5]))
        for tid, t in self.sparse.items():
            out.append((f"table {t.name!r}", t.status))
        if self.bucket is not None:
            out += [("dense step", w) for w in self.bucket.status_words()]
        return out

    def _poll_status(self) -> None:
        pend = getattr(self, "_status_pending", None)
        if pend is not None:
            event, host, words = pend
            if not event.query():
                return
            self._status_pending = None
            codes = host.tolist()
            bad = [(label, code, w) for (label, w), code in zip(words, codes) if code != 0]
            if bad:
                for _, _, w in bad:
                    w.zero_()
                raise C.KrakenError("; ".join(f"{label}: {C.error_message(code)} (code {code})" for label, code, _ in bad))
        if self._steps % max(1, int(getattr(self.cfg, "status_poll_interval", 8))) != 0:
            return
        words = self._status_words()
        if not words:
            return
        host = getattr(self, "_status_host", None)
        if host is None or host.numel() < len(words):
            host = self._status_host = torch.zeros(max(16, 2 * len(words)), dtype=torch.int32).pin_memory()
        for k, (_, w) in enumerate(words):
            host[k:k + 1].copy_(w, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._status_pending = (ev, host[:len(words)], words)

    def _ensure_room(self, table_id: int, n_ids: int) -> None:
        """Makes sure the shard can take the rows this lookup may create BEFORE the kernels run (growth
        by ``end_step`` reacts one step late: a first batch larger than the free slots would otherwise
        hit the probe limit and come back as kTableFull).  A host-side upper bound of the row count is
        kept per table; only when it nears the load limit is the exact counter read (one synchronisation)."""
        if torch.cuda.is_current_stream_capturing():
            return
        t = self.sparse[table_id]
        ch = self.channels.get(table_id)
        inflow = n_ids * self.world  # worst case: every rank's ids of this call belong to this shard
        if ch is not None:
            # no more than the exchange buffers admit (world x cap_s), and with a uniform owner hash about
            # 1 / world of every rank's unique ids - twice that is reserved; a shard that still runs full
            # reports kTableFull and is grown by end_step()
            n_ids = min(n_ids, ch.cap_u)
            inflow = min(self.world * ch.cap_s, 2 * n_ids) if self.world > 1 else n_ids
        hi = getattr(t, "rows_hi", 0) + inflow
        if hi > 0.6 * t.capacity:
            exact = t.num_rows()
            hi = exact + inflow
            if hi > 0.6 * t.capacity:
                t.reserve(hi)
        t.rows_hi = hi

    def check(self) -> None:
        """Raises if any kernel recorded an error (synchronises)."""
        for ch in list(self.channels.values()) + list(self.nccl_channels.values()) + list(self.group_channels.values()):
            ch.check()
        for t in self.sparse.values():
            t.check()
        if self.bucket is not None:
            self.bucket.check()

    def kernel_launches(self) -> int:
        from ..ops import counters
        n = sum(ch.launches for ch in self.channels.values()) + counters.launches()
        n += sum(ch.launches for ch in self.group_channels.values())
        n += sum(ch.local.launches for ch in self.nccl_channels.values())
        if self.bucket is not None:
            n += self.bucket.launches
        return n

    # ------------------------------------------------------------------ checkpoint glue
    def export_dense(self, table_id: int) -> dict:
        return self._ensure_bucket().export_table(table_id, self._table(table_id, "dense").shape)

    def import_dense(self, table_id: int, name: str, value: dict) -> None:
        self._ensure_bucket().import_table(table_id, value)

    def dense_owner(self, table_id: int) -> int:
        return table_id % self.world

    def export_sparse(self, table_id: int) -> dict:
        return self.sparse[table_id].export()

    def import_sparse(self, table_id: int, cols: dict) -> None:
        self.sparse[table_id].import_rows(cols["ids"], cols["vals"], cols["states"], cols["states_i"])

    def save_sparse_streamed(self, table_id: int, out_dir: str, info: TableInfo) -> dict:
        return self.sparse[table_id].save_streamed(out_dir, info.init_type, info.init_conf)

    def import_sparse_routed(self, table_id: int, name: str, dirs: Sequence[str], chunk_rows: int = 1 << 21) -> int:
        """Checkpoint load for GPU shards.  This rank reads ALL rows of the shard files in ``dirs`` (its 1 / world
        share of the checkpoint) and sends every row to the rank that owns it under the current placement
        (device-side owner computation, one all-to-all per chunk over NCCL); owners insert what they receive.
        Fixed-layout files are read chunk by chunk with ``SparseChunkReader`` into two sets of pinned staging
        buffers: a reader thread fills one set (preads + column extraction on 8 threads) while the other set is
        uploaded, routed and inserted, so the host never holds more than two chunks and pays the page faults of
        its buffers once.  Anything else - a file the reference wrote with per-row state sets - goes through the
        general reader as a whole.  Collective: ranks with fewer chunks take part with empty ones.
        Replaces "every rank parses every file and drops (world - 1) / world of it"."""
        import threading
        t = self.sparse[table_id]
        salt = self._salt(table_id)
        dev = self.device
        # sources: ("file", reader, a, b) rows [a, b) of a fixed-layout file; ("mem", columns, a, b) parsed columns
        sources = []
        skeys, ikeys = set(), set()
        for d in dirs:
            rd = C.SparseChunkReader(d, name)
            if not rd.exists:
                continue
            if rd.fast and rd.dim == t.dim:
                skeys.update(int(k) for k in rd.state_types)
                ikeys.update(int(k) for k in rd.int_state_types)
                sources += [("file", rd, a, min(a + chunk_rows, int(rd.rows))) for a in range(0, int(rd.rows), chunk_rows)]
                continue
            cols = C.ckpt_load_sparse(d, name)
            if cols is not None and cols["ids"].numel() > 0:
                skeys.update(int(k) for k in cols["states"])
                ikeys.update(int(k) for k in cols["states_i"])
                n = int(cols["ids"].numel())
                sources += [("mem", cols, a, min(a + chunk_rows, n)) for a in range(0, n, chunk_rows)]
        skeys, ikeys = sorted(skeys), sorted(ikeys)
        rounds = len(sources)
        if self.world > 1:
            # every rank must know the same column set and the same number of rounds
            meta = torch.zeros(2 + 16, dtype=torch.int64, device=dev)
            meta[0] = rounds
            for k in skeys:
                meta[2 + k] = 1
            for k in ikeys:
                meta[2 + 8 + k] = 1
            dist.all_reduce(meta, op=dist.ReduceOp.MAX, group=self.group)
            rounds = int(meta[0].item())
            flags = meta[2:].tolist()
            skeys = [k for k in range(8) if flags[k]]
            ikeys = [k for k in range(8) if flags[8 + k]]

        file_rows = max([b - a for kind, _, a, b in sources if kind == "file"], default=0)
        stage = []
        if file_rows:
            stage = [{"ids": torch.empty(file_rows, dtype=torch.int64, pin_memory=True),
                      "vals": torch.empty((file_rows, t.dim), dtype=torch.float32, pin_memory=True),
                      "f": {k: torch.empty((file_rows, t.dim), dtype=torch.float32, pin_memory=True) for k in skeys},
                      "i": {k: torch.empty(file_rows, dtype=torch.int64, pin_memory=True) for k in ikeys},
                      "free": None} for _ in range(2)]
        fill_result = {}

        def fill(r: int) -> None:
            """Reader thread: source r -> staging set r % 2 (file sources only)."""
            kind, src, a, b = sources[r]
            buf = stage[r % 2]
            if buf["free"] is not None:
                buf["free"].synchronize()      # the uploads of round r - 2 have left this set
            ok = src.read_into(a, b - a, buf["ids"], buf["vals"], [buf["f"][int(k)] for k in src.state_types],
                               [buf["i"][int(k)] for k in src.int_state_types])
            fill_result[r] = bool(ok)

        def start_fill(r: int):
            if r < len(sources) and sources[r][0] == "file":
                th = threading.Thread(target=fill, args=(r,), daemon=True)
                th.start()
                return th
            return None

        read = 0
        pending = start_fill(0)
        for r in range(rounds):
            if r < len(sources):
                kind, src, a, b = sources[r]
                m = b - a
                if kind == "file":
                    pending.join()
                    if not fill_result.pop(r):
                        raise C.KrakenError(f"{name}: a row of the checkpoint file deviates from the file's layout")
                    buf = stage[r % 2]
                    pending = start_fill(r + 1)      # the next chunk is read while this one is uploaded and inserted
                    have_f, have_i = {int(k) for k in src.state_types}, {int(k) for k in src.int_state_types}
                    ids = buf["ids"][:m].to(dev, non_blocking=True)
                    vals = buf["vals"][:m].to(dev, non_blocking=True)
                    states = {k: (buf["f"][k][:m].to(dev, non_blocking=True) if k in have_f
                                  else torch.zeros((m, t.dim), device=dev)) for k in skeys}
                    states_i = {k: (buf["i"][k][:m].to(dev, non_blocking=True) if k in have_i
                                    else torch.zeros(m, dtype=torch.int64, device=dev)) for k in ikeys}
                    buf["free"] = torch.cuda.Event()
                    buf["free"].record()
                else:
                    if pending is None:
                        pending = start_fill(r + 1)
                    ids = src["ids"][a:b].to(dev, non_blocking=True)
                    vals = src["vals"][a:b].to(dev, non_blocking=True)
                    states = {k: (src["states"][k][a:b].to(dev, non_blocking=True) if k in src["states"]
                                  else torch.zeros((m, t.dim), device=dev)) for k in skeys}
                    states_i = {k: (src["states_i"][k][a:b].to(dev, non_blocking=True) if k in src["states_i"]
                                    else torch.zeros(m, dtype=torch.int64, device=dev)) for k in ikeys}
                read += m
            else:
                ids = torch.empty(0, dtype=torch.int64, device=dev)
                vals = torch.empty((0, t.dim), device=dev)
                states = {k: torch.empty((0, t.dim), device=dev) for k in skeys}
                states_i = {k: torch.empty(0, dtype=torch.int64, device=dev) for k in ikeys}
            if self.world > 1:
                owners = C.owner_of_cuda(ids, salt, self.owner_world).long() if ids.numel() else torch.empty(0, dtype=torch.long, device=dev)
                order = torch.argsort(owners, stable=True)
                send = torch.bincount(owners, minlength=self.world)
                recv = torch.empty_like(send)
                dist.all_to_all_single(recv, send, group=self.group)
                sc, rc = send.tolist(), recv.tolist()

                def a2a(x, width):
                    out = torch.empty((sum(rc), width) if width else (sum(rc),), dtype=x.dtype, device=dev)
                    dist.all_to_all_single(out, x[order].contiguous(), rc, sc, group=self.group)
                    return out

                ids = a2a(ids, 0)
                vals = a2a(vals, t.dim)
                states = {k: a2a(v, t.dim) for k, v in states.items()}
                states_i = {k: a2a(v, 0) for k, v in states_i.items()}
            if ids.numel():
                t.import_rows(ids, vals, states, states_i)
        if pending is not None:
            pending.join()
        torch.cuda.synchronize(dev)   # the staging buffers are freed below: their last uploads must have finished
        return read

    def stop(self) -> None:
        if self.stopped:
            return
        if self.profiler is not None:
            self.profiler.close()
        torch.cuda.synchronize()
        failure = None
        try:
            self.check()  # an error recorded after the last poll must not disappear with the engine
        except C.KrakenError as e:
            failure = e
        if self.world > 1:
            dist.barrier(group=self.group)
        for ch in list(self.channels.values()) + list(self.nccl_channels.values()) + list(self.group_channels.values()):
            ch.close()
        self.nccl_channels.clear()
        self.group_channels.clear()
        if self.bucket is not None:
            self.bucket.close()
        self.channels.clear()
        self.bucket = None
        from ..ops import mlp as fused_mlp
        fused_mlp.set_deferred_join(False)
        fused_mlp.set_grad_ready_callback(None)
        super().stop()
        if failure is not None:
            raise failure
