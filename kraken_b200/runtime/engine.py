"""Process-global training engine: what ``kraken.pytorch.initialize`` creates.

The reference runs three kinds of processes (scheduler, parameter servers,
workers; kraken/scheduler/scheduler.cc, kraken/ps/ps.cc, kraken/worker/emitter.cc).
Here every rank is worker and shard at once (one process per GPU, or per CPU
rank), so the scheduler's table registry becomes a deterministic per-rank
registry: all ranks register the same tables in the same order and therefore
agree on ids without a round trip.  Two engines share that registry:

* ``CpuEngine``  - C++ CpuShard per rank, gloo all-to-all between ranks;
* ``GpuEngine``  - GPU hash-table shards, fused peer-memory kernels.

Both expose the functions of the reference's ``kraken_native`` module
(kraken/pytorch/py/py.cc:42-97) with the same names and argument order.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from .._native import C


@dataclass
class EngineConfig:
    backend: str = "auto"            # "cpu" | "gpu" | "auto" ("remote" / "zmq" are chosen by the address given to initialize)
    emitter_type: object = None      # C.EmitterType
    life_span: int = 1000
    eta: float = 0.75
    seed: int = 0
    table_capacity: int = 1 << 20    # initial slots per GPU shard (tables grow)
    max_ids_per_call: int = 0        # 0: sized from the first call (2x headroom)
    max_unique_per_call: int = 0     # 0: same as max_ids_per_call; smaller saves exchange-buffer memory
    async_push: bool = False         # TCP deployment: pushes are applied by a background thread, the caller does not wait (a pull may be one push stale)
    long_id_streams: bool = False    # GPU engine: a pull / push longer than the exchange buffers runs as several rounds (the ranks agree on the count: one small all-reduce per call)
    max_per_owner_per_call: int = 0  # 0: same as max_unique_per_call; unique ids one rank may send to one owner
    spin_limit: int = 1 << 22        # polls before a device-side wait gives up
    saved_dir: str = ""
    max_save_count: int = 3
    owner_salt_per_table: bool = False
    exchange: str = "fused"          # "fused": peer-memory kernels; "nccl": torch.distributed collectives (baseline)
    compress: object = None          # TCP deployment: CompressType of worker<->server bodies (None / kNo = off)
    dense_bucket_elems: int = 1 << 21  # GPU engine: dense tables are grouped into buckets of at least this many
                                       # elements; with overlap_dense_step each is stepped as soon as its gradients exist
    status_poll_interval: int = 8    # GPU engine: steps between asynchronous reads of the kernels' error words
    overlap_dense_step: bool = False  # run the fused dense step on the MLP backward's side stream, beside the
                                      # sparse backward + push (needs: nothing reads the MLP's .grad before step())


@dataclass
class TableInfo:
    id: int
    name: str
    kind: str                        # "dense" | "sparse"
    shape: Sequence[int] = ()
    dimension: int = 0
    init_type: object = None
    init_conf: Dict[str, str] = field(default_factory=dict)
    dtype: object = torch.float32    # what the caller registered; shards always hold float32


def _env_int(name: str, default: int) -> int:
    try:
        return int(os.environ.get(name, default))
    except ValueError:
        return default


class Engine:
    """Registry + API surface; the data plane is in the subclasses."""

    def __init__(self, cfg: EngineConfig, rank: int, world: int, group=None) -> None:
        self.cfg = cfg
        self.rank = rank
        self.world = world
        self.group = group
        self.model_name: Optional[str] = None
        self.optim_type = None
        self.optim_conf: Dict[str, str] = {}
        self.tables: Dict[int, TableInfo] = {}
        self.name_to_id: Dict[str, int] = {}
        self.lr = 0.0
        self.router = C.Router.for_ranks(world)
        self.stopped = False

    # ------------------------------------------------------------------ registry
    def init_model(self, model_name: str, optim_type, optim_conf: Optional[Dict[str, str]] = None) -> None:
        optim_conf = dict(optim_conf or {})
        if self.model_name is not None:
            # idempotent like Scheduler::InitModel (kraken/scheduler/scheduler.cc:154-190)
            return
        self.model_name = model_name
        self.optim_type = optim_type
        self.optim_conf = optim_conf
        self._on_init_model()

    def update_lr(self, lr: float) -> None:
        self.lr = float(lr)
        self._on_update_lr()

    def _need_model(self) -> None:
        if self.model_name is None:
            raise C.KrakenError("model not initialized: call init_model first")

    def _new_id(self, table_id: Optional[int]) -> int:
        """Ids are dense in registration order unless a checkpoint dictates one."""
        if table_id is None:
            table_id = 0
            while table_id in self.tables:
                table_id += 1
        elif table_id in self.tables:
            raise C.KrakenError(f"table id {table_id} is already taken")
        return int(table_id)

    def register_dense_table(self, name: str, val: torch.Tensor, table_id: Optional[int] = None) -> int:
        self._need_model()
        if name in self.name_to_id:
            info = self.tables[self.name_to_id[name]]
            if info.kind != "dense" or tuple(info.shape) != tuple(val.shape):
                raise C.KrakenError(f"dense table {name!r} is already registered with another type or shape")
            return info.id
        tid = self._new_id(table_id)
        info = TableInfo(id=tid, name=name, kind="dense", shape=tuple(val.shape),
                         dtype=val.dtype if val.is_floating_point() else torch.float32)
        self.tables[tid] = info
        self.name_to_id[name] = tid
        self._on_register_dense(info, val)
        return tid

    def register_sparse_table(self, name: str, dimension: int, dtype, init_type, init_conf: Dict[str, str],
                              table_id: Optional[int] = None) -> int:
        self._need_model()
        # Shards hold float32 rows and state whatever the caller asks for; float64 / float16 / bfloat16
        # tables are converted where values leave or enter the engine (pytorch/native.py).
        if dtype not in (torch.float32, torch.float64, torch.float16, torch.bfloat16, None):
            raise C.KrakenError("sparse tables are float32, float64, float16 or bfloat16")
        if name in self.name_to_id:
            info = self.tables[self.name_to_id[name]]
            if info.kind != "sparse" or info.dimension != int(dimension) or info.init_type != init_type:
                raise C.KrakenError(f"sparse table {name!r} is already registered with another dimension or initializer")
            return info.id
        tid = self._new_id(table_id)
        info = TableInfo(id=tid, name=name, kind="sparse", dimension=int(dimension), init_type=init_type,
                         init_conf=dict(init_conf), dtype=dtype or torch.float32)
        self.tables[tid] = info
        self.name_to_id[name] = tid
        self._on_register_sparse(info)
        return tid

    def _table(self, table_id: int, kind: str) -> TableInfo:
        info = self.tables.get(int(table_id))
        if info is None:
            raise C.KrakenError(f"table {table_id} does not exist")
        if info.kind != kind:
            raise C.KrakenError(f"table {table_id} is not a {kind} table")
        return info

    def model_meta(self):
        m = C.ModelMeta()
        m.name = self.model_name or ""
        m.optim_type = self.optim_type
        m.optim_conf = dict(self.optim_conf)
        tables = {}
        for tid, info in self.tables.items():
            t = C.TableMeta()
            t.id = tid
            t.name = info.name
            if info.kind == "dense":
                t.table_type = C.TableType.kDense
                t.shape = list(info.shape)
            else:
                t.table_type = C.TableType.kSparse
                t.dimension = info.dimension
                t.init_type = info.init_type
                t.init_conf = dict(info.init_conf)
            tables[tid] = t
        m.tables = tables
        return m

    # ------------------------------------------------------------------ combined calls
    def combine_pull_dense_table(self, table_ids: Sequence[int]) -> List[torch.Tensor]:
        return [self.pull_dense_table(t) for t in table_ids]

    def combine_pull_sparse_table(self, table_ids: Sequence[int], indices: Sequence[torch.Tensor]) -> List[torch.Tensor]:
        if len(table_ids) != len(indices):
            raise C.KrakenError("table_ids and indices differ in length")
        return [self.pull_sparse_table(t, i) for t, i in zip(table_ids, indices)]

    def combine_push_sparse_table(self, table_ids: Sequence[int], indices: Sequence[torch.Tensor],
                                  grads: Sequence[torch.Tensor]) -> None:
        if not (len(table_ids) == len(indices) == len(grads)):
            raise C.KrakenError("table_ids, indices and grads differ in length")
        # reverse order: the matching pull of the last table is the freshest ticket
        for t, i, g in reversed(list(zip(table_ids, indices, grads))):
            self.push_sparse_table(t, i, g)

    # ------------------------------------------------------------------ hooks for subclasses
    def _on_init_model(self) -> None: ...
    def _on_update_lr(self) -> None: ...
    def _on_register_dense(self, info: TableInfo, val: torch.Tensor) -> None: ...
    def _on_register_sparse(self, info: TableInfo) -> None: ...

    def end_step(self) -> None:
        """Called by Optimizer.step() after the dense update: housekeeping between steps."""

    def stop(self) -> None:
        self.stopped = True
