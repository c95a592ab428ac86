"""GPU-resident sparse-table shard and its exchange channel.

``GpuSparseTable`` is this rank's part of one sparse table: an open-addressing
hash table over int64 ids whose slots index structure-of-arrays slabs (values,
optimizer state, step counters) in HBM.  It replaces the reference server's
lock-striped skip lists (kraken/ps/sparse_table.h:28,
kraken/common/parallel_skip_list.h:19-21).

``SparseChannel`` owns the symmetric buffers through which the ranks exchange
ids, rows and gradients for that table, and drives the fused pull / push kernel
sequence (csrc/cuda/sparse.cu).  It replaces the client data plane of
kraken/worker/emitter.cc:123-183 (pull) and :491-550 (push).

Pull and push are collective: every rank of the group must call them in the
same order, with its own local ids.  Nothing here synchronises the host.
"""
from __future__ import annotations

import math
import os
from typing import Dict, Optional

import torch

from .._native import C
from .symm import Layout, SymmetricArena

_EMPTY = -1  # 0xFFFF_FFFF_FFFF_FFFF as int64: the reserved "free slot" key
DEFAULT_SPIN = 1 << 22


def _next_pow2_bits(n: int) -> int:
    return max(4, int(math.ceil(math.log2(max(2, n)))))


class GpuSparseTable:
    """One rank's shard of a sparse table."""

    def __init__(self, table_id: int, name: str, dim: int, init_type, init_conf: Dict[str, str], optim_type,
                 optim_conf: Dict[str, str], seed: int, capacity: int, world: int, device: torch.device) -> None:
        self.table_id = table_id
        self.name = name
        self.dim = int(dim)
        self.init_type = init_type
        self.init_conf = dict(init_conf)
        self.optim_type = optim_type
        self.optim_conf = dict(optim_conf)
        self.optim_info = C.parse_optim(optim_type, optim_conf)
        self.optim = C.make_optim(optim_type, optim_conf)
        self.init = C.parse_init(init_type, init_conf)
        self.seed_key = C.seed_key(seed, table_id)
        self.world = world
        self.device = device
        self.bits = _next_pow2_bits(capacity)
        self.size = torch.zeros(1, dtype=torch.int32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self._size_host = torch.zeros(1, dtype=torch.int32).pin_memory() if device.type == "cuda" else None
        self._size_event: Optional[torch.cuda.Event] = None
        self._alloc(self.bits)

    # ------------------------------------------------------------------ storage
    def _alloc(self, bits: int) -> None:
        self.generation = getattr(self, "generation", 0) + 1  # bumps whenever the slabs move: cached descriptors are stale
        cap = 1 << bits
        dev = self.device
        info = self.optim_info
        self.bits = bits
        self.keys = torch.full((cap,), _EMPTY, dtype=torch.int64, device=dev)
        self.val = torch.zeros((cap, self.dim), dtype=torch.float32, device=dev)
        self.slabs = []
        for k in range(3):
            if info["slabs"][k]:
                fill = info["initial_accumulator_value"] if (info["type"] == 0 and k == 0) else 0.0
                self.slabs.append(torch.full((cap, self.dim), fill, dtype=torch.float32, device=dev))
            else:
                self.slabs.append(None)
        self.steps = torch.zeros(cap, dtype=torch.int32, device=dev) if info["needs_steps"] else None
        self.lead = torch.zeros(cap, dtype=torch.int64, device=dev) if self.world > 1 else None
        self._host = C.make_table(self.keys, self.val, self.slabs[0], self.slabs[1], self.slabs[2], self.steps,
                                  self.lead, self.size, self.status, bits, self.dim, self.init[0], self.init[1],
                                  self.init[2], self.seed_key)

    @property
    def capacity(self) -> int:
        return 1 << self.bits

    def host(self):
        return self._host

    # ------------------------------------------------------------------ maintenance
    def num_rows(self) -> int:
        """Occupied slots (synchronises)."""
        return int(self.size.item())

    def check(self) -> None:
        code = int(self.status.item())
        if code != 0:
            self.status.zero_()
            raise C.KrakenError(f"table {self.name!r}: {C.error_message(code)} (code {code})")

    def export(self, filter_mode: int = 0, salt: int = 0, world: int = 1, rank: int = 0, min_steps: int = 0):
        """Copies the rows that pass the filter out of the table.

        filter_mode 0 = all rows, 1 = rows owned by ``rank`` under a modulo-``world``
        placement, 2 = rows NOT owned by it, 3 = rows updated at least ``min_steps`` times.
        Returns a dict of device tensors: ids [n], vals [n, dim], states {StateType: [n, dim]},
        states_i {0: steps [n]}.
        """
        count = torch.zeros(1, dtype=torch.int32, device=self.device)
        C.table_export(self._host, filter_mode, salt, world, rank, min_steps, None, None, None, None, None, None, count)
        n = int(count.item())
        dev = self.device
        ids = torch.empty(n, dtype=torch.int64, device=dev)
        vals = torch.empty((n, self.dim), dtype=torch.float32, device=dev)
        souts = [torch.empty((n, self.dim), dtype=torch.float32, device=dev) if s is not None else None
                 for s in self.slabs]
        steps = torch.empty(n, dtype=torch.int32, device=dev) if self.steps is not None else None
        if n > 0:
            C.table_export(self._host, filter_mode, salt, world, rank, min_steps, ids, vals, souts[0], souts[1],
                           souts[2], steps, count)
        states = {}
        for k in range(3):
            if souts[k] is not None:
                states[int(self.optim_info["slab_state_types"][k])] = souts[k]
        states_i = {0: steps.to(torch.int64)} if steps is not None else {}
        return {"dim": self.dim, "ids": ids, "vals": vals, "states": states, "states_i": states_i}

    def save_streamed(self, out_dir: str, init_type, init_conf, chunk_rows: int = 1 << 21, threads: int = 0) -> dict:
        """Writes this shard's rows as ``<name>.sparse`` in the reference's file format without a host-side copy
        of the table: for each of the file's 8 slots (id % 8) the matching rows are compacted on the device,
        ordered by id (as unsigned numbers) with a device sort, and streamed in chunks through two pinned
        buffers on a copy stream to a multi-threaded writer (csrc/core/checkpoint.cc: SparseStreamWriter), so the
        copy of chunk k + 1 overlaps the formatting and writing of chunk k.  Returns {"rows", "bytes"}."""
        info = self.optim_info
        threads = threads or max(2, min(8, (os.cpu_count() or 8)))   # 16 threads were no faster than 8 on a 16-core host
        cols = sorted((int(info["slab_state_types"][k]), k) for k in range(3) if self.slabs[k] is not None)
        int_types = [0] if self.steps is not None else []
        w = C.SparseStreamWriter(out_dir, self.table_id, self.name, self.dim, init_type, dict(init_conf),
                                 [st for st, _ in cols], int_types, threads)
        dev = self.device
        copy_stream = torch.cuda.Stream(device=dev)
        n_cols = 1 + len(cols)
        pinned = [{"ids": torch.empty(chunk_rows, dtype=torch.int64, pin_memory=True),
                   "f": [torch.empty((chunk_rows, self.dim), dtype=torch.float32, pin_memory=True) for _ in range(n_cols)],
                   "steps": torch.empty(chunk_rows, dtype=torch.int64, pin_memory=True), "event": None} for _ in range(2)]
        total = 0
        flip = torch.tensor(-(1 << 63), dtype=torch.int64, device=dev)
        for slot in range(8):
            part = self.export(filter_mode=4, world=8, rank=slot)
            n = int(part["ids"].numel())
            w.begin_slot(n)
            if n == 0:
                continue
            order = torch.argsort(part["ids"] ^ flip)   # ascending as uint64
            fcols = [part["vals"]] + [part["states"][st] for st, _ in cols]
            steps = part["states_i"][0] if self.steps is not None else None
            pending = None
            for k, a in enumerate(range(0, n, chunk_rows)):
                sel = order[a:a + chunk_rows]
                m = int(sel.numel())
                buf = pinned[k % 2]
                staged = [part["ids"].index_select(0, sel)] + [c.index_select(0, sel) for c in fcols]
                staged_steps = steps.index_select(0, sel) if steps is not None else None
                copy_stream.wait_stream(torch.cuda.current_stream(dev))
                with torch.cuda.stream(copy_stream):
                    buf["ids"][:m].copy_(staged[0], non_blocking=True)
                    for dst, src in zip(buf["f"], staged[1:]):
                        dst[:m].copy_(src, non_blocking=True)
                        src.record_stream(copy_stream)
                    staged[0].record_stream(copy_stream)
                    if staged_steps is not None:
                        buf["steps"][:m].copy_(staged_steps, non_blocking=True)
                        staged_steps.record_stream(copy_stream)
                    ev = torch.cuda.Event()
                    ev.record(copy_stream)
                if pending is not None:        # write the previous chunk while this one crosses PCIe
                    self._append_chunk(w, *pending)
                pending = (buf, m, ev, steps is not None)
            if pending is not None:
                self._append_chunk(w, *pending)
            total += n
            del part, order, fcols
        w.close()
        return {"rows": total, "bytes": int(w.bytes_written())}

    @staticmethod
    def _append_chunk(w, buf, m, event, has_steps) -> None:
        event.synchronize()
        w.append(buf["ids"][:m], buf["f"][0][:m], [c[:m] for c in buf["f"][1:]], [buf["steps"][:m]] if has_steps else [])

    def import_rows(self, ids: torch.Tensor, vals: torch.Tensor, states: Optional[dict] = None,
                    states_i: Optional[dict] = None) -> None:
        """Inserts (or overwrites) rows with the given values and optimizer state."""
        n = int(ids.numel())
        if n == 0:
            return
        total = self.num_rows() + n
        self.reserve(total)
        self.rows_hi = max(getattr(self, "rows_hi", 0), total)  # host-side upper bound used by the engine's growth check
        dev = self.device
        ids = ids.to(dev, torch.int64).contiguous()
        vals = vals.to(dev, torch.float32).contiguous()
        sl = [None, None, None]
        for k in range(3):
            st = int(self.optim_info["slab_state_types"][k])
            if self.slabs[k] is not None and states and st in states:
                sl[k] = states[st].to(dev, torch.float32).contiguous()
        steps = None
        if self.steps is not None and states_i and 0 in states_i:
            steps = states_i[0].to(dev, torch.int32).contiguous()
        C.table_import(self._host, ids, vals, sl[0], sl[1], sl[2], steps)

    def reserve(self, rows: int, max_load: float = 0.6) -> bool:
        """Grows (rehashes) so that ``rows`` rows stay below ``max_load``; True if it grew."""
        need_bits = _next_pow2_bits(int(rows / max_load) + 1)
        if need_bits <= self.bits:
            return False
        old = self.export()
        self.size.zero_()
        self._alloc(need_bits)
        C.table_import(self._host, old["ids"], old["vals"],
                       *[old["states"].get(int(self.optim_info["slab_state_types"][k])) if self.slabs[k] is not None
                         else None for k in range(3)],
                       old["states_i"][0].to(torch.int32) if self.steps is not None else None)
        return True

    def poll_growth(self, max_load: float = 0.6) -> bool:
        """Non-blocking load-factor check: looks at the size counter copied out
        during the previous call and starts the next copy.  Call between steps."""
        grew = False
        if self._size_host is not None:
            if self._size_event is not None and self._size_event.query():
                rows = int(self._size_host[0])
                # the sample is a step or two old: leave room for what arrives at the pace seen since the last one
                pace = max(0, rows - getattr(self, "_rows_seen", rows))
                self._rows_seen = rows
                if rows + 2 * pace > max_load * self.capacity:
                    grew = self.reserve(int((rows + 2 * pace) * 2))
                self._size_event = None
            if self._size_event is None:
                self._size_host.copy_(self.size, non_blocking=True)
                self._size_event = torch.cuda.Event()
                self._size_event.record()
        return grew

    def evict(self, min_steps: int) -> int:
        """Drops the rows updated fewer than ``min_steps`` times by rebuilding the
        table from the survivors; returns how many rows were dropped."""
        before = self.num_rows()
        keep = self.export(filter_mode=3, min_steps=min_steps)
        C.table_clear(self._host)
        self.val.zero_()
        for k, s in enumerate(self.slabs):
            if s is not None:
                s.fill_(self.optim_info["initial_accumulator_value"] if (self.optim_info["type"] == 0 and k == 0)
                        else 0.0)
        self.import_rows(keep["ids"], keep["vals"], keep["states"], keep["states_i"])
        return before - int(keep["ids"].numel())

    def lookup(self, ids: torch.Tensor):
        """(rows [n, dim], found [n]) for ids on this shard, without inserting."""
        return C.table_lookup(self._host, ids.to(self.device, torch.int64).contiguous())


class Ticket:
    """Identifies one pull so that the matching push can reuse its dedup result
    and the slots the owners resolved."""

    __slots__ = ("channel", "serial", "n", "bag_offsets", "weights", "mean", "bag_mean", "slots")

    def __init__(self, channel, serial, n, bag_offsets, weights, mean, bag_mean, slots=None):
        self.slots = slots  # in-place pulls: table slot of every unique entry (rows are the table's value slab)
        self.channel = channel
        self.serial = serial
        self.n = n
        self.bag_offsets = bag_offsets
        self.weights = weights
        self.mean = mean
        self.bag_mean = bag_mean


class SparseChannel:
    """Exchange buffers + kernel sequence of one table."""

    def __init__(self, table: GpuSparseTable, rank: int, world: int, max_ids: int, group=None,
                 spin_limit: int = DEFAULT_SPIN, owner_salt: int = 0, alias_peers: bool = False,
                 max_unique: int = 0, max_per_owner: int = 0) -> None:
        """max_ids bounds the occurrences of one call, max_unique (default: max_ids) the unique ids
        among them, max_per_owner (default: max_unique) the unique ids one rank sends to ONE owner.  The
        receive buffer is sized by max_unique; the peer inboxes and the gradient inbox hold
        world x max_per_owner entries - with a uniform owner hash about max_unique / world per owner are
        expected, so a bound of two or three times that saves most of the worst-case memory.  A call that
        exceeds a bound is reported as kInboxOverflow, never written out of bounds."""
        self.table = table
        self.rank = rank
        self.world = world
        self.group = group
        self.spin = int(spin_limit)
        self.salt = int(owner_salt)
        self.cap = int(max_ids)
        self.cap_u = int(max_unique) if max_unique and max_unique < max_ids else int(max_ids)
        self.cap_s = int(max_per_owner) if max_per_owner and max_per_owner < self.cap_u else self.cap_u
        dim = table.dim
        dev = table.device

        lay = Layout()
        lay.add("inbox_ids", (world, self.cap_s), torch.int64)
        lay.add("inbox_meta", (world, 2), torch.int32)
        lay.add("rows_recv", (self.cap_u, dim), torch.float32)
        lay.add("inbox_grad", (world, self.cap_s, dim), torch.float32)
        lay.add("flag_req", (world,), torch.int32)
        lay.add("flag_rsp", (world,), torch.int32)
        lay.add("flag_push", (world,), torch.int32)
        self.arena = SymmetricArena(lay, rank, world, group, alias_peers)
        self.lay = C.ChanLayout()
        for name in ("inbox_ids", "inbox_meta", "rows_recv", "inbox_grad", "flag_req", "flag_rsp", "flag_push"):
            setattr(self.lay, name, lay.offset(name))
        self.lay.capS = self.cap_s
        self.lay.capU = self.cap_u

        self.ctrl = torch.zeros(C.CTRL_INTS, dtype=torch.int32, device=dev)  # csrc/cuda/kernels.h: Ctrl
        self.hbits = _next_pow2_bits(2 * self.cap)
        # dedup scratch set: entries of (key, position | winner << 32); every key is free between calls
        self.hkeys = torch.zeros((1 << self.hbits, 2), dtype=torch.int64, device=dev)
        self.hkeys[:, 0] = _EMPTY
        self.slot_of = torch.zeros(self.cap, dtype=torch.int32, device=dev)
        self.cnt = torch.zeros(world, dtype=torch.int32, device=dev)
        self._own_off = torch.zeros(world + 1, dtype=torch.int32, device=dev)
        self._own_uniq = torch.zeros(self.cap_u, dtype=torch.int64, device=dev)
        self._own_inv = torch.zeros(self.cap, dtype=torch.int32, device=dev)
        self.off, self.uniq, self.inv = self._own_off, self._own_uniq, self._own_inv
        self.rows_recv = self.arena.window("rows_recv")
        self.slot_cache = torch.full((world * self.cap_s,), -1, dtype=torch.int32, device=dev)
        self.ugrad = torch.zeros((self.cap_u, dim), dtype=torch.float32, device=dev)
        self.serial = 0
        self.launches = 0  # kernels launched through this channel (for accounting)
        self._wait = 1 if world > 1 else 0  # the one-warp rendezvous kernels exist only between GPUs
        self.owner_world = world            # rows live on ranks 0 .. owner_world - 1 (smaller after a live reshard)

    # ------------------------------------------------------------------ helpers
    def _lookup_phase(self, ids: torch.Tensor, insert: bool, share_from: Optional["SparseChannel"] = None) -> int:
        """Dedup + dispatch + owner-side probe.  ``share_from``: another channel that has just
        deduplicated the SAME ids with the same owner salt; its unique list and occurrence map
        are used instead of computing them again."""
        n = int(ids.numel())
        if n > self.cap:
            raise C.KrakenError(f"table {self.table.name!r}: {n} ids in one call exceed the channel capacity "
                                f"{self.cap}; raise max_ids_per_call")
        h, lay, ctrl, tbl = self.arena.heap, self.lay, self.ctrl, self.table.host()
        if share_from is not None and share_from.salt == self.salt and share_from.world == self.world:
            self.off, self.uniq, self.inv = share_from.off, share_from.uniq, share_from.inv
            C.pull_dispatch(h, lay, ctrl, self.uniq, self.off, n)
            self.launches += 1
        else:
            # the dedup's second kernel also sends the unique ids to their owners' inboxes
            self.off, self.uniq, self.inv = self._own_off, self._own_uniq, self._own_inv
            C.dedup_bucketize(ids, self.world, self.salt, self.hkeys, self.slot_of, self.hbits,
                              self.cnt, self.off, self.uniq, self.inv, self.ctrl[4:5], self.cap_u, h, lay, ctrl,
                              self.owner_world)
            self.launches += 2
        C.pull_probe(h, lay, ctrl, tbl, self.slot_cache, insert, self.spin)
        self.launches += 1 + self._wait  # (request wait +) probe, which also initialises the rows it creates
        self.serial += 1
        self.last_n = n
        return n

    def last_exchange(self) -> dict:
        """Counters of the latest lookup (synchronises): occurrences, unique ids, how many of them
        other ranks own, and the bytes that crossed NVLink for them in each phase, per direction
        (ids out and rows in for a pull, gradient rows out for a push)."""
        n = getattr(self, "last_n", 0)
        off = self.off.cpu().tolist()
        unique = int(off[self.world])
        own = int(off[self.rank + 1] - off[self.rank])
        remote = unique - own
        row_bytes = self.table.dim * 4
        return {"occurrences": n, "unique": unique, "unique_ratio": unique / n if n else 0.0, "unique_remote": remote,
                "pull_bytes_out": remote * 8, "pull_bytes_in": remote * row_bytes, "push_bytes_out": remote * row_bytes}

    def pull_unique(self, ids: torch.Tensor, share_from: Optional["SparseChannel"] = None, in_place: bool = False):
        """Pull that stops before the expansion: returns (unique rows buffer [cap, dim],
        occurrence -> unique map [n], ticket).  The rows belong to the channel and are
        overwritten by its next pull; a consumer kernel reads them through the map.

        ``in_place`` (honoured on single-GPU jobs): no copy of the rows is made; the first result is
        the table's value slab and ``ticket.slots[u]`` is the slab row of unique entry ``u``.
        Worth it for small batches only: a consumer that visits every occurrence then reads
        scattered table rows instead of a compact buffer that fits in L2."""
        ids = ids.reshape(-1)
        n = self._lookup_phase(ids, insert=True, share_from=share_from)
        if in_place and self.world == 1:
            return self.table.val, self.inv, Ticket(self, self.serial, n, None, None, False, None, self.slot_cache)
        C.pull_gather(self.arena.heap, self.lay, self.ctrl, self.table.host(), self.slot_cache)
        if self.world > 1:
            C.pull_wait(self.arena.heap, self.lay, self.ctrl, self.spin)
        self.launches += 1 + self._wait
        return self.rows_recv, self.inv, Ticket(self, self.serial, n, None, None, False, None)

    def push_accumulated(self, lr: torch.Tensor, ticket: Ticket) -> None:
        """Push for gradients that a fused kernel has already summed per unique id into
        ``self.ugrad`` (the pull's ticket must still be current)."""
        if ticket.channel is not self or ticket.serial != self.serial:
            raise C.KrakenError("push_accumulated needs the ticket of this channel's latest pull")
        h, lay, ctrl, tbl = self.arena.heap, self.lay, self.ctrl, self.table.host()
        C.push_dispatch(h, lay, ctrl, self.ugrad, self.off, ticket.n, self.table.dim)
        C.push_apply(h, lay, ctrl, tbl, self.slot_cache, self.table.optim, lr, self.spin)
        self.launches += 2 + 2 * self._wait  # dispatch, (push wait, merge,) update
        self.serial += 1

    # ------------------------------------------------------------------ pull
    def pull(self, ids: torch.Tensor, bag_offsets: Optional[torch.Tensor] = None,
             weights: Optional[torch.Tensor] = None, mean: bool = False, bag_mean: Optional[torch.Tensor] = None,
             patch_value: float = 0.0, out: Optional[torch.Tensor] = None):
        """Looks up (inserting unseen ids) and returns (rows, ticket).

        Without ``bag_offsets`` rows is [n, dim], one per id.  With ``bag_offsets``
        ([k + 1], int64) rows is [k, dim]: each bag's rows pooled by sum, or mean
        where ``mean`` / ``bag_mean[b]`` says so; empty bags give ``patch_value``.
        """
        ids = ids.reshape(-1)
        n = self._lookup_phase(ids, insert=True)
        h, lay, ctrl, tbl = self.arena.heap, self.lay, self.ctrl, self.table.host()
        dim = self.table.dim
        C.pull_gather(h, lay, ctrl, tbl, self.slot_cache)
        rows = (int(bag_offsets.numel()) - 1) if bag_offsets is not None else n
        if out is None:
            out = torch.empty((rows, dim), dtype=torch.float32, device=self.table.device)
        C.pull_combine(h, lay, ctrl, self.inv, n, dim, bag_offsets, weights, mean, bag_mean, patch_value, out,
                       self.spin)
        self.launches += 2 + self._wait  # gather, (response wait,) combine
        return out, Ticket(self, self.serial, n, bag_offsets, weights, mean, bag_mean)

    # ------------------------------------------------------------------ push
    def push(self, grads: torch.Tensor, lr: torch.Tensor, ticket: Optional[Ticket] = None,
             ids: Optional[torch.Tensor] = None, bag_offsets: Optional[torch.Tensor] = None,
             weights: Optional[torch.Tensor] = None, mean: bool = False,
             bag_mean: Optional[torch.Tensor] = None) -> None:
        """Sums the gradients of duplicate ids, sends them to the owners and runs
        the optimizer there.  With the ticket of the latest pull of this channel
        the dedup result and the owners' slots are reused; otherwise ``ids`` are
        looked up again (an id the table does not hold is kSparseIdNotExist)."""
        if ticket is not None and ticket.channel is self and ticket.serial == self.serial:
            n = ticket.n
            bag_offsets, weights, mean, bag_mean = ticket.bag_offsets, ticket.weights, ticket.mean, ticket.bag_mean
        else:
            if ids is None:
                raise C.KrakenError("push without a current ticket needs the ids")
            n = self._lookup_phase(ids.reshape(-1), insert=False)
        h, lay, ctrl, tbl = self.arena.heap, self.lay, self.ctrl, self.table.host()
        dim = self.table.dim
        grads = grads.reshape(-1, dim)
        if grads.dtype != torch.float32 or not grads.is_contiguous():
            grads = grads.to(torch.float32).contiguous()
        C.push_scatter(grads, self.inv, n, dim, bag_offsets, weights, mean, bag_mean, self.ugrad)
        C.push_dispatch(h, lay, ctrl, self.ugrad, self.off, n, dim)
        C.push_apply(h, lay, ctrl, tbl, self.slot_cache, self.table.optim, lr, self.spin)
        self.launches += 3 + 2 * self._wait  # scatter, dispatch, (push wait, merge,) update
        # A push consumes the pull's bookkeeping: a second push needs a new lookup.
        self.serial += 1

    # ------------------------------------------------------------------ status
    def check(self) -> None:
        code = int(self.ctrl[4].item())
        if code != 0:
            self.ctrl[4].zero_()
            raise C.KrakenError(f"channel of table {self.table.name!r}: {C.error_message(code)} (code {code})")
        self.table.check()

    def close(self) -> None:
        self.arena.close()


class GroupChannel:
    """One exchange for several tables of the same row width (csrc/cuda/sparse_group.cu).

    The ids of the tables travel as one concatenated list: one dedup keyed by (table, id), one
    dispatch, one owner-side probe, one gather and one push sequence serve the whole group - what the
    reference does with its combined requests (kraken/worker/emitter.cc:185-278, :552-632;
    kraken/ps/ps_op.cc:370-387, :456-469).  ``pull`` returns one [n_total, dim] buffer holding the rows of
    every table's ids back to back (split it per table); ``push`` takes the gradients in the same layout.
    Collective like SparseChannel: every rank calls with the same tables in the same order.
    """

    def __init__(self, tables, rank: int, world: int, max_ids: int, group=None, spin_limit: int = DEFAULT_SPIN,
                 salts=None, alias_peers: bool = False, max_unique: int = 0) -> None:
        dims = {t.dim for t in tables}
        if len(dims) != 1:
            raise C.KrakenError("the tables of a group must have the same dimension")
        self.tables = list(tables)
        self.T = len(self.tables)
        self.dim = self.tables[0].dim
        self.rank, self.world, self.group = rank, world, group
        self.spin = int(spin_limit)
        self.cap = int(max_ids)
        self.cap_u = int(max_unique) if max_unique and max_unique < max_ids else int(max_ids)
        dev = self.tables[0].device
        self.device = dev
        T, dim = self.T, self.dim

        lay = Layout()
        lay.add("inbox_ids", (world, self.cap_u), torch.int64)
        lay.add("inbox_meta", (world, 2), torch.int32)
        lay.add("inbox_tcnt", (world, T + 1), torch.int32)
        lay.add("rows_recv", (self.cap_u, dim), torch.float32)
        lay.add("inbox_grad", (world, self.cap_u, dim), torch.float32)
        lay.add("flag_req", (world,), torch.int32)
        lay.add("flag_rsp", (world,), torch.int32)
        lay.add("flag_push", (world,), torch.int32)
        self.arena = SymmetricArena(lay, rank, world, group, alias_peers)
        self.lay = C.ChanLayout()
        for name in ("inbox_ids", "inbox_meta", "inbox_tcnt", "rows_recv", "inbox_grad", "flag_req", "flag_rsp",
                     "flag_push"):
            setattr(self.lay, name, lay.offset(name))
        self.lay.capS = self.cap_u
        self.lay.capU = self.cap_u

        self.ctrl = torch.zeros(C.CTRL_INTS, dtype=torch.int32, device=dev)
        self.salts = torch.tensor([int(x) for x in (salts or [0] * T)], dtype=torch.int64, device=dev)
        self.snap_t = torch.zeros(world * (T + 1), dtype=torch.int32, device=dev)
        self.slot_of = torch.zeros(self.cap, dtype=torch.int32, device=dev)
        self.cnt = torch.zeros(world * T, dtype=torch.int32, device=dev)
        self.off = torch.zeros(world + 1, dtype=torch.int32, device=dev)
        self.uniq = torch.zeros(self.cap_u, dtype=torch.int64, device=dev)
        self.inv = torch.zeros(self.cap, dtype=torch.int32, device=dev)
        self.rows_recv = self.arena.window("rows_recv")
        self.slot_cache = torch.full((world * self.cap_u,), -1, dtype=torch.int32, device=dev)
        self.ttab = torch.zeros(world * self.cap_u, dtype=torch.int16, device=dev)
        self.ugrad = torch.zeros((self.cap_u, dim), dtype=torch.float32, device=dev)
        self.hkeys = None           # dedup scratch, one region per table, sized on first use
        self._shape_sig = None      # ids per table of the call the descriptors were built for
        self._views_sig = None      # generations of the tables the device-side descriptors describe
        self.owner_world = world    # rows live on ranks 0 .. owner_world - 1 (smaller after a live reshard)
        self.table_views = None
        self.serial = 0
        self.launches = 0

    # ------------------------------------------------------------------ descriptors
    def _describe(self, counts) -> None:
        """Device-side description of a call's shape (ids per table) - rebuilt only when it changes."""
        sig = tuple(int(c) for c in counts)
        if sig == self._shape_sig:
            return
        if torch.cuda.is_current_stream_capturing():
            raise C.KrakenError("the number of ids per table changed inside a CUDA-graph capture")
        occ, base, bits, pos = [0], [], [], 0
        for c in sig:
            occ.append(occ[-1] + c)
            b = _next_pow2_bits(2 * max(c, 1))
            base.append(pos)
            bits.append(b)
            pos += 1 << b
        dev = self.device
        self.occ_start = torch.tensor(occ, dtype=torch.int32, device=dev)
        self.region_base = torch.tensor(base, dtype=torch.int32, device=dev)
        self.region_bits = torch.tensor(bits, dtype=torch.int32, device=dev)
        if self.hkeys is None or self.hkeys.shape[0] < pos:
            self.hkeys = torch.zeros((pos, 2), dtype=torch.int64, device=dev)
            self.hkeys[:, 0] = _EMPTY
        self._shape_sig = sig

    def _refresh_views(self) -> None:
        sig = tuple(t.generation for t in self.tables)
        if sig == self._views_sig:
            return
        host = C.group_table_views([t.host() for t in self.tables])
        if self.table_views is None:
            self.table_views = host.to(self.device)
        else:
            self.table_views.copy_(host)   # same device buffer: launches captured in a CUDA graph stay valid
        self._views_sig = sig

    # ------------------------------------------------------------------ exchange
    def _lookup_phase(self, ids_cat: torch.Tensor, counts, insert: bool) -> int:
        n = int(ids_cat.numel())
        if n > self.cap:
            raise C.KrakenError(f"{n} ids in one combined call exceed the channel capacity {self.cap}; "
                                "raise max_ids_per_call")
        self._describe(counts)
        self._refresh_views()
        h, lay, ctrl = self.arena.heap, self.lay, self.ctrl
        C.group_dedup_dispatch(ids_cat, self.occ_start, self.region_base, self.region_bits, self.salts, self.world,
                               self.hkeys, self.slot_of, self.cnt, self.off, self.uniq, self.inv, self.ctrl[4:5],
                               self.cap_u, h, lay, ctrl, self.owner_world)
        C.group_probe(h, lay, ctrl, self.table_views, self.T, self.dim, self.snap_t, self.slot_cache, self.ttab,
                      insert, self.spin)
        self.launches += 5  # memset is not counted: insert, finalize + dispatch, request wait, probe (+ init)
        self.serial += 1
        self.last_n = n
        return n

    def pull(self, ids_cat: torch.Tensor, counts, bag_offsets: Optional[torch.Tensor] = None,
             weights: Optional[torch.Tensor] = None, bag_mean: Optional[torch.Tensor] = None,
             patch_value: float = 0.0):
        """ids_cat: the tables' ids back to back, counts[t] of them for table t.  Returns (rows, ticket):
        rows is [n_total, dim], or [k_total, dim] pooled per bag when ``bag_offsets`` (over the concatenated
        list) is given - ``bag_mean[b]`` selects mean pooling per bag."""
        n = self._lookup_phase(ids_cat.reshape(-1), counts, insert=True)
        h, lay, ctrl = self.arena.heap, self.lay, self.ctrl
        C.group_gather(h, lay, ctrl, self.table_views, self.dim, self.slot_cache, self.ttab)
        rows = (int(bag_offsets.numel()) - 1) if bag_offsets is not None else n
        out = torch.empty((rows, self.dim), dtype=torch.float32, device=self.device)
        C.pull_combine(h, lay, ctrl, self.inv, n, self.dim, bag_offsets, weights, False, bag_mean, patch_value, out,
                       self.spin)
        self.launches += 2 + (1 if self.world > 1 else 0)
        return out, Ticket(self, self.serial, n, bag_offsets, weights, False, bag_mean)

    def push(self, grads_cat: torch.Tensor, lr: torch.Tensor, ticket: Optional[Ticket] = None,
             ids_cat: Optional[torch.Tensor] = None, counts=None) -> None:
        """Gradients in the layout ``pull`` returned.  With the ticket of this channel's latest pull the
        dedup result and the owners' slots are reused; otherwise the ids are looked up again (an id a table
        does not hold is kSparseIdNotExist)."""
        bag_offsets = weights = bag_mean = None
        if ticket is not None and ticket.channel is self and ticket.serial == self.serial:
            n = ticket.n
            bag_offsets, weights, bag_mean = ticket.bag_offsets, ticket.weights, ticket.bag_mean
        else:
            if ids_cat is None or counts is None:
                raise C.KrakenError("a combined push without a current ticket needs the ids")
            n = self._lookup_phase(ids_cat.reshape(-1), counts, insert=False)
        h, lay, ctrl = self.arena.heap, self.lay, self.ctrl
        grads = grads_cat.reshape(-1, self.dim)
        if grads.dtype != torch.float32 or not grads.is_contiguous():
            grads = grads.to(torch.float32).contiguous()
        C.push_scatter(grads, self.inv, n, self.dim, bag_offsets, weights, False, bag_mean, self.ugrad)
        C.push_dispatch(h, lay, ctrl, self.ugrad, self.off, n, self.dim)
        C.group_push_apply(h, lay, ctrl, self.table_views, self.dim, self.slot_cache, self.ttab, self.tables[0].optim,
                           lr, self.spin)
        self.launches += 3 + (2 if self.world > 1 else 0)
        self.serial += 1

    def check(self) -> None:
        code = int(self.ctrl[4].item())
        if code != 0:
            self.ctrl[4].zero_()
            names = ", ".join(repr(t.name) for t in self.tables[:4]) + (", ..." if self.T > 4 else "")
            raise C.KrakenError(f"combined channel of tables {names}: {C.error_message(code)} (code {code})")
        for t in self.tables:
            t.check()

    def close(self) -> None:
        self.arena.close()
