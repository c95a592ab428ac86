"""Dense parameter tables on the GPUs: one flat, bucketed buffer.

All dense tables of a model are packed back to back (each starting on a
256-element boundary) into one fp32 parameter buffer and one gradient buffer
that live in symmetric memory.  Rank r owns slice r of the flat range together
with the optimizer state of that slice (ZeRO-1 style); ``step()`` launches the
fused reduce-scatter + optimizer + all-gather kernel (csrc/cuda/dense.cu).

``param_view`` / ``grad_view`` hand out the tensors that a model's
``nn.Parameter.data`` / ``.grad`` alias, so the backward pass accumulates
straight into the exchange buffer and the updated values appear in place: the
reference's per-table push RPC, server update and per-step pull
(kraken/pytorch/optimizer.py:141-173) cost no copy here.

With ``emitter_type == kDCT`` the gradient is sparsified per table before it
crosses NVLink (top ``1 - eta`` by magnitude, threshold refreshed every
``life_span`` steps, the rest kept as error feedback), as in
kraken/worker/dct_emitter.cc:16-43.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .._native import C
from .symm import Layout, SymmetricArena
from .sparse_shard import DEFAULT_SPIN

CHUNK = 256
DCT_MIN_SIZE = 256  # tables smaller than this always travel whole (dct_emitter.cc:18-20)


class DenseBucket:
    def __init__(self, tables: Sequence[Tuple[int, int]], optim_type, optim_conf: Dict[str, str], rank: int,
                 world: int, device: torch.device, group=None, dct: bool = False, life_span: int = 1000,
                 eta: float = 0.75, spin_limit: int = DEFAULT_SPIN) -> None:
        """tables: (table_id, numel) in registration order."""
        self.rank, self.world, self.device, self.group = rank, world, device, group
        self.optim_info = C.parse_optim(optim_type, optim_conf)
        self.optim = C.make_optim(optim_type, optim_conf)
        self.spin = int(spin_limit)
        self.dct = bool(dct)
        self.life_span = int(life_span)
        self.eta = float(eta)

        self.table_ids: List[int] = []
        self.offsets: Dict[int, Tuple[int, int]] = {}
        pos = 0
        chunk_table: List[int] = []
        for idx, (tid, numel) in enumerate(tables):
            self.table_ids.append(tid)
            self.offsets[tid] = (pos, int(numel))
            nchunks = (int(numel) + CHUNK - 1) // CHUNK
            chunk_table += [idx] * nchunks
            pos += nchunks * CHUNK
        unit = world * CHUNK
        self.n_pad = max(unit, (pos + unit - 1) // unit * unit)
        chunk_table += [-1] * (self.n_pad // CHUNK - len(chunk_table))
        self.slice = self.n_pad // world

        lay = Layout()
        lay.add("grad", (self.n_pad,), torch.float32)
        lay.add("param", (self.n_pad,), torch.float32)
        lay.add("flag_grad", (world,), torch.int32)
        lay.add("flag_done", (world,), torch.int32)
        lay.add("coo_cnt", (world,), torch.int32)
        if self.dct:
            lay.add("coo_idx", (self.n_pad,), torch.int32)
            lay.add("coo_val", (self.n_pad,), torch.float32)
        self.arena = SymmetricArena(lay, rank, world, group)
        self.lay = C.DenseLayout()
        for name in lay.entries:
            setattr(self.lay, name, lay.offset(name))
        self.bases = [self.arena.heap.peer_ptr(p) for p in range(world)]

        self.grad = self.arena.window("grad")
        self.param = self.arena.window("param")
        self.ctrl = torch.zeros(C.DENSE_CTRL_INTS, dtype=torch.int32, device=device)  # csrc/cuda/dense_kernels.h: DenseCtrl
        self.chunk_table = torch.tensor(chunk_table, dtype=torch.int32, device=device)
        n_tables = max(1, len(self.table_ids))
        self.table_steps = torch.zeros(n_tables, dtype=torch.int32, device=device)
        self.table_active = torch.ones(n_tables, dtype=torch.uint8, device=device)
        self._active_host = [True] * n_tables
        info = self.optim_info
        self.state: List[Optional[torch.Tensor]] = []
        for k in range(3):
            if info["slabs"][k]:
                fill = info["initial_accumulator_value"] if (info["type"] == 0 and k == 0) else 0.0
                self.state.append(torch.full((self.slice,), fill, dtype=torch.float32, device=device))
            else:
                self.state.append(None)
        self.acc = torch.zeros(self.slice, dtype=torch.float32, device=device) if self.dct else None
        if self.dct:
            self.residual = torch.zeros(self.n_pad, dtype=torch.float32, device=device)
            self.tau = torch.zeros(n_tables, dtype=torch.float32, device=device)
            self.hist = torch.zeros(1024, dtype=torch.int32, device=device)
            self.prefix = torch.zeros(2, dtype=torch.int32, device=device)
            self.dct_step = 0
        self.launches = 0

    # ------------------------------------------------------------------ views
    def param_view(self, table_id: int, shape: Sequence[int]) -> torch.Tensor:
        off, numel = self.offsets[table_id]
        return self.param[off:off + numel].view(*shape)

    def grad_view(self, table_id: int, shape: Sequence[int]) -> torch.Tensor:
        off, numel = self.offsets[table_id]
        return self.grad[off:off + numel].view(*shape)

    def set_active(self, active: Sequence[bool]) -> None:
        active = list(active)
        if active != self._active_host:
            self._active_host = active
            self.table_active.copy_(torch.tensor(active, dtype=torch.uint8))

    # ------------------------------------------------------------------ step
    def step(self, lr: torch.Tensor, grad_scale: float = 1.0) -> None:
        """Collective.  Consumes the gradient buffer (zero afterwards) and leaves
        the updated parameters in every rank's ``param`` buffer."""
        if self.dct:
            C.dct_accumulate(self.grad, self.residual)
            if self.dct_step % self.life_span == 0:
                for idx, tid in enumerate(self.table_ids):
                    off, numel = self.offsets[tid]
                    if numel < DCT_MIN_SIZE:
                        continue  # tau stays 0: the table travels whole
                    k = int(numel * (1.0 - self.eta))
                    if k < 1:
                        raise C.KrakenError("DCT keeps no element: eta too close to 1")
                    C.dct_select_tau(self.grad[off:off + numel], k, self.hist, self.prefix, self.tau[idx:idx + 1])
                    self.launches += 9
            C.dct_compact(self.bases, self.rank, self.lay, self.n_pad, self.residual, self.tau, self.chunk_table)
            self.dct_step += 1
            self.launches += 2
        C.dense_step(self.bases, self.rank, self.lay, self.ctrl, self.n_pad, self.state[0], self.state[1],
                     self.state[2], self.acc, self.chunk_table, self.table_steps, self.table_active, self.optim, lr,
                     float(grad_scale), self.dct, self.spin)
        # between GPUs: rendezvous, (COO gather,) update, wait for the owners, zero; one GPU: (COO gather,) update
        self.launches += (4 if self.world > 1 else 1) + (1 if self.dct else 0)

    def check(self) -> None:
        code = int(self.ctrl[3].item())
        if code != 0:
            self.ctrl[3].zero_()
            raise C.KrakenError(f"dense step: {C.error_message(code)} (code {code})")

    # ------------------------------------------------------------------ checkpoint
    def export_table(self, table_id: int, shape: Sequence[int]) -> dict:
        """Value + optimizer state of one table, gathered from the owning slices (collective)."""
        off, numel = self.offsets[table_id]
        out = {"val": self.param[off:off + numel].detach().clone().view(*shape).cpu(), "states": {}, "states_i": {}}
        idx = self.table_ids.index(table_id)
        steps = int(self.table_steps[idx].item())
        if steps > 0:
            for k in range(3):
                if self.state[k] is None:
                    continue
                full = self._gather_state(k)
                out["states"][int(self.optim_info["slab_state_types"][k])] = full[off:off + numel].view(*shape).cpu()
            if self.optim_info["needs_steps"]:
                out["states_i"][0] = steps
        return out

    def _gather_state(self, k: int) -> torch.Tensor:
        if self.world == 1:
            return self.state[k]
        import torch.distributed as dist

        parts = [torch.empty_like(self.state[k]) for _ in range(self.world)]
        dist.all_gather(parts, self.state[k], group=self.group)
        return torch.cat(parts)

    def import_table(self, table_id: int, value: dict) -> None:
        off, numel = self.offsets[table_id]
        self.param[off:off + numel].copy_(value["val"].reshape(-1).to(self.device, torch.float32))
        lo, hi = self.rank * self.slice, (self.rank + 1) * self.slice
        a, b = max(off, lo), min(off + numel, hi)
        for k in range(3):
            st = int(self.optim_info["slab_state_types"][k])
            if self.state[k] is None or st not in value.get("states", {}) or a >= b:
                continue
            src = value["states"][st].reshape(-1).to(self.device, torch.float32)
            self.state[k][a - lo:b - lo].copy_(src[a - off:b - off])
        if 0 in value.get("states_i", {}):
            self.table_steps[self.table_ids.index(table_id)] = int(value["states_i"][0])

    def close(self) -> None:
        self.arena.close()


class BucketSet:
    """The dense tables of a model split into several ``DenseBucket``s, in registration order.

    Each bucket has its own symmetric arena, flags and optimizer-state slices, so it can be stepped
    (reduce-scatter + optimizer + all-gather, one fused kernel sequence) as soon as ITS gradients are
    complete, while the backward pass still computes the gradients of the layers in front of it: the
    reference pushes every dense gradient from a per-parameter hook during backward
    (kraken/pytorch/optimizer.py:115-121,141-149); here the unit is a bucket of at least
    ``bucket_elems`` elements so that small tables share one launch sequence.  The interface is that
    of a single ``DenseBucket``; ``step`` steps whatever has not been stepped since the previous ``step``.
    """

    def __init__(self, tables: Sequence[Tuple[int, int]], optim_type, optim_conf: Dict[str, str], rank: int,
                 world: int, device: torch.device, group=None, dct: bool = False, life_span: int = 1000,
                 eta: float = 0.75, spin_limit: int = DEFAULT_SPIN, bucket_elems: int = 1 << 21) -> None:
        groups: List[List[Tuple[int, int]]] = [[]]
        size = 0
        for tid, numel in tables:
            groups[-1].append((tid, numel))
            size += int(numel)
            if size >= bucket_elems:
                groups.append([])
                size = 0
        if not groups[-1] and len(groups) > 1:
            groups.pop()
        self.buckets = [DenseBucket(g, optim_type, optim_conf, rank, world, device, group, dct, life_span, eta,
                                    spin_limit) for g in groups]
        self.table_ids: List[int] = [tid for g in groups for tid, _ in g]
        self.bucket_of: Dict[int, int] = {tid: k for k, g in enumerate(groups) for tid, _ in g}
        self.n_pad = sum(b.n_pad for b in self.buckets)
        self.world, self.rank, self.device = world, rank, device
        self._stepped = [False] * len(self.buckets)

    # ------------------------------------------------------------------ views
    def param_view(self, table_id: int, shape: Sequence[int]) -> torch.Tensor:
        return self.buckets[self.bucket_of[table_id]].param_view(table_id, shape)

    def grad_view(self, table_id: int, shape: Sequence[int]) -> torch.Tensor:
        return self.buckets[self.bucket_of[table_id]].grad_view(table_id, shape)

    def grads(self) -> List[torch.Tensor]:
        return [b.grad for b in self.buckets]

    def set_active(self, active: Sequence[bool]) -> None:
        active = list(active)
        pos = 0
        for b in self.buckets:
            n = len(b.table_ids)
            b.set_active(active[pos:pos + n])
            pos += n

    # ------------------------------------------------------------------ step
    def step_bucket(self, k: int, lr: torch.Tensor, grad_scale: float = 1.0) -> None:
        """Steps bucket k now, on the current stream (collective: every rank steps its buckets in the same order)."""
        if not self._stepped[k]:
            self.buckets[k].step(lr, grad_scale)
            self._stepped[k] = True

    def step(self, lr: torch.Tensor, grad_scale: float = 1.0) -> None:
        """Steps every bucket that ``step_bucket`` has not stepped since the last call, last bucket first (the
        order in which a backward pass completes them), and starts a new round."""
        for k in range(len(self.buckets) - 1, -1, -1):
            self.step_bucket(k, lr, grad_scale)
        self._stepped = [False] * len(self.buckets)

    @property
    def launches(self) -> int:
        return sum(b.launches for b in self.buckets)

    def status_words(self) -> List[torch.Tensor]:
        return [b.ctrl[3:4] for b in self.buckets]

    def check(self) -> None:
        for b in self.buckets:
            b.check()

    # ------------------------------------------------------------------ checkpoint
    def export_table(self, table_id: int, shape: Sequence[int]) -> dict:
        return self.buckets[self.bucket_of[table_id]].export_table(table_id, shape)

    def import_table(self, table_id: int, value: dict) -> None:
        self.buckets[self.bucket_of[table_id]].import_table(table_id, value)

    def close(self) -> None:
        for b in self.buckets:
            b.close()
