"""Function-level API with the names of the reference's ``kraken_native``
extension module (kraken/pytorch/py/py.cc:20-97), bound to a process-global
engine instead of a ZeroMQ worker.

``initialize`` keeps the reference signature ``(s_addr, emitter_type, life_span,
eta)``.  ``s_addr`` selects the backend: ``"gpu"`` / ``"cpu"`` (optionally with
``://`` and anything after it), while any other address - such as the
``host:port`` a reference script passes - means "auto": GPUs if present;
``tcp://host:port`` connects to a running ``scheduler_server`` (multi-process CPU
deployment, ``kraken_b200.launch``).  When
the process runs under ``torchrun`` (RANK / WORLD_SIZE set) the ranks form one
job: NCCL for the GPU engine, gloo for the CPU engine.
"""
from __future__ import annotations

import os
import re
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from .._native import C
from ..runtime.engine import Engine, EngineConfig

OptimType = C.OptimType
InitializerType = C.InitializerType
EmitterType = C.EmitterType
KrakenError = C.KrakenError


class CompressType:
    """Name quirk kept for source compatibility: the reference exports its wire
    CompressType {kNo, kSnappy} under these two names (kraken/pytorch/py/py.cc:34-36)."""
    kDefault = 0
    kDCT = 1


_engine: Optional[Engine] = None
_owns_process_group = False


def engine() -> Engine:
    if _engine is None:
        raise KrakenError("kraken is not initialized: call initialize() first")
    return _engine


def is_initialized() -> bool:
    return _engine is not None


def initialize(s_addr: str = "auto", emitter_type=EmitterType.kDefault, life_span: int = 1000, eta: float = 0.75,
               **options) -> None:
    """Creates the engine once per process (later calls are ignored, like the
    reference's call_once, kraken/pytorch/py/pytorch.cc:21-26).

    Extra keyword options: seed, table_capacity, max_ids_per_call, spin_limit,
    saved_dir, max_save_count, backend ("cpu" | "gpu").
    """
    global _engine, _owns_process_group
    if _engine is not None:
        return
    from ..utils.log import configure as _configure_logging
    _configure_logging()
    backend = options.pop("backend", None)
    if backend is None:
        head = (s_addr or "auto").split("://")[0].lower()
        backend = head if head in ("cpu", "gpu", "zmq") else ("remote" if head == "tcp" else "auto")
        if backend == "auto" and re.fullmatch(r"[^:/\s]+:\d{1,5}", s_addr or ""):
            backend = "remote"     # "host:port", the reference's form of a scheduler address
    if backend == "auto":
        backend = "gpu" if torch.cuda.is_available() else "cpu"
    cfg = EngineConfig(backend=backend, emitter_type=emitter_type, life_span=int(life_span), eta=float(eta))
    cfg.saved_dir = os.environ.get("KRAKEN_SAVED_DIR", "")
    for k, v in options.items():
        if not hasattr(cfg, k):
            raise KrakenError(f"unknown initialize option {k!r}")
        setattr(cfg, k, v)

    if backend == "zmq":
        # this framework's worker on a cluster of the REFERENCE's scheduler and servers (its ZeroMQ wire protocol)
        from ..runtime.zmq_client import ZmqRemoteEngine
        _engine = ZmqRemoteEngine(cfg, s_addr.split("://", 1)[-1])
        return
    if backend == "remote":
        # multi-process CPU deployment: s_addr = "tcp://host:port" of a running scheduler_server
        from ..runtime.remote import RemoteEngine
        _engine = RemoteEngine(cfg, s_addr.split("://", 1)[-1])
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if backend == "gpu":
        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local % max(1, torch.cuda.device_count()))
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if backend == "gpu":
            dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
        else:
            dist.init_process_group("gloo")
        _owns_process_group = True
    if dist.is_initialized():
        world, rank = dist.get_world_size(), dist.get_rank()

    if backend == "gpu":
        from ..runtime.gpu_engine import GpuEngine
        _engine = GpuEngine(cfg, rank, world)
    else:
        from ..runtime.cpu_engine import CpuEngine
        _engine = CpuEngine(cfg, rank, world)


def stop(keep_process_group: bool = False) -> None:
    """Shuts the engine down.  ``keep_process_group``: leave a torch.distributed group that
    ``initialize`` created in place, so that a later ``initialize`` in the same process reuses it
    (a second NCCL rendezvous on the launcher's store is not possible once rank 0 has left it)."""
    global _engine, _owns_process_group
    if _engine is None:
        return
    _engine.stop()
    _engine = None
    if _owns_process_group and dist.is_initialized() and not keep_process_group:
        dist.destroy_process_group()
        _owns_process_group = False


def init_model(model_name: str, optim_type, optim_conf: Optional[Dict[str, str]] = None) -> None:
    engine().init_model(model_name, optim_type, optim_conf or {})


def update_lr(lr: float) -> None:
    engine().update_lr(lr)


def register_dense_table(name: str, val: torch.Tensor) -> int:
    return engine().register_dense_table(name, val)


def register_sparse_table(name: str, dimension: int, dtype, init_type, init_conf: Dict[str, str]) -> int:
    return engine().register_sparse_table(name, dimension, dtype, init_type, init_conf)


def _as_registered(table_id: int, t: torch.Tensor) -> torch.Tensor:
    """Values leave the engine in the dtype the table was registered with (shards hold float32)."""
    info = engine().tables.get(table_id)
    want = getattr(info, "dtype", torch.float32) if info is not None else torch.float32
    return t if t.dtype == want else t.to(want)


def pull_dense_table(table_id: int) -> torch.Tensor:
    return _as_registered(table_id, engine().pull_dense_table(table_id))


def combine_pull_dense_table(table_ids: Sequence[int]) -> List[torch.Tensor]:
    return [_as_registered(i, t) for i, t in zip(table_ids, engine().combine_pull_dense_table(list(table_ids)))]


def push_dense_table(table_id: int, grad: torch.Tensor) -> None:
    engine().push_dense_table(table_id, grad)


def pull_sparse_table(table_id: int, indices: torch.Tensor) -> torch.Tensor:
    return _as_registered(table_id, engine().pull_sparse_table(table_id, indices))


def combine_pull_sparse_table(table_ids: Sequence[int], indices: Sequence[torch.Tensor]) -> List[torch.Tensor]:
    outs = engine().combine_pull_sparse_table(list(table_ids), list(indices))
    return [_as_registered(i, t) for i, t in zip(table_ids, outs)]


def push_sparse_table(table_id: int, indices: torch.Tensor, grad: torch.Tensor) -> None:
    engine().push_sparse_table(table_id, indices, grad)


def combine_push_sparse_table(table_ids: Sequence[int], indices: Sequence[torch.Tensor],
                              grads: Sequence[torch.Tensor]) -> None:
    engine().combine_push_sparse_table(list(table_ids), list(indices), list(grads))


def try_save_model() -> bool:
    eng = engine()
    if hasattr(eng, "check"):
        eng.check()  # a table that recorded an error must not be written out as if it were sound
    if hasattr(eng, "try_save_model"):
        return eng.try_save_model()
    from ..checkpoint.manager import save_model
    return save_model(eng)


def try_load_model_blocked(load_dir: str) -> bool:
    eng = engine()
    if hasattr(eng, "try_load_model_blocked"):
        return eng.try_load_model_blocked(load_dir)
    from ..checkpoint.manager import load_model
    return load_model(eng, load_dir)


def jagged_sum_forward(values, offsets, patch_value, weights=None):
    return C.jagged_sum_forward(values, offsets, patch_value, weights)


def jagged_sum_backward(offsets, grads, weights=None):
    return C.jagged_sum_backward(offsets, grads, weights)


def jagged_mean_forward(values, offsets, patch_value, weights=None):
    return C.jagged_mean_forward(values, offsets, patch_value, weights)


def jagged_mean_backward(offsets, grads, weights=None):
    return C.jagged_mean_backward(offsets, grads, weights)
