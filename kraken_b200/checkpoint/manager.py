"""Checkpoint save / load orchestration in the reference's directory layout.

    <saved_dir>/shard_<rank>/<YYYY-MM-DD-HH-MM-SS>/{router,model}.{json,binary}, *.dense, *.sparse

Every rank writes its own shard directory: the same router and model metadata,
the dense tables it is the designated writer of, and its rows of every sparse
table (kraken/checkpoint/checkpoint_exec.cc:246-377).  Loading discovers the
newest snapshot of every shard, rebuilds the registry from ``model.binary`` and
keeps of every row only those the CURRENT placement assigns to this rank, so a
checkpoint written by N shards - by this framework or by the reference - loads
into M shards (kraken/checkpoint/checkpoint_exec.cc:379-521,
kraken/checkpoint/checkpoint.cc:587-649).
"""
from __future__ import annotations

import logging
import os
import time
from typing import Dict

import torch
import torch.distributed as dist

from .._native import C

log = logging.getLogger("kraken_b200")


def _barrier(engine) -> None:
    if engine.world > 1:
        dist.barrier(group=engine.group)


def save_model(engine, saved_dir: str = "") -> bool:
    """Collective.  Returns False when no directory is configured or no model exists."""
    saved_dir = saved_dir or engine.cfg.saved_dir
    if not saved_dir or engine.model_name is None:
        return False
    t0 = time.time()
    out = C.ckpt_prepare_save_dir(saved_dir, engine.rank, engine.cfg.max_save_count)
    C.ckpt_save_router(out, engine.router)
    C.ckpt_save_model(out, engine.model_meta())
    rows = nbytes = 0
    for tid, info in sorted(engine.tables.items()):
        if info.kind == "dense":
            value = engine.export_dense(tid)  # collective on the GPU engine
            if engine.dense_owner(tid) == engine.rank:
                C.ckpt_save_dense(out, tid, info.name, value)
        elif hasattr(engine, "save_sparse_streamed"):
            # GPU shards: device-side ordering, chunks through pinned buffers, multi-threaded writer
            done = engine.save_sparse_streamed(tid, out, info)
            rows += done["rows"]
            nbytes += done["bytes"]
        else:
            cols = engine.export_sparse(tid)
            ids = cols["ids"].cpu()
            rows += int(ids.numel())
            C.ckpt_save_sparse(out, tid, info.name, info.dimension, info.init_type, info.init_conf, ids,
                               cols["vals"].cpu(), {k: v.cpu() for k, v in cols["states"].items()},
                               {k: v.cpu() for k, v in cols["states_i"].items()})
    _barrier(engine)
    dt = time.time() - t0
    log.info("rank %d saved %d sparse rows to %s in %.2fs%s", engine.rank, rows, out, dt,
             f" ({nbytes / dt / 1e9:.2f} GB/s)" if nbytes else "")
    engine.last_checkpoint = {"op": "save", "rows": rows, "bytes": nbytes, "seconds": dt}
    return True


def load_model(engine, load_dir: str) -> bool:
    """Collective.  Must run before the Optimizer is built; its registrations then
    find the loaded tables (registration by name is idempotent)."""
    if engine.model_name is not None:
        return True  # already initialised: nothing is loaded (kraken/scheduler/scheduler.cc:379-384)
    shard_dirs: Dict[int, str] = C.ckpt_latest_shard_dirs(load_dir)
    if not shard_dirs:
        return False
    first = shard_dirs[min(shard_dirs)]
    meta = C.ckpt_load_model(first)
    old_router = C.ckpt_load_router(first)
    log.info("loading model %r written by %d shard(s); saved router: %s", meta.name, len(shard_dirs), old_router)
    engine.init_model(meta.name, meta.optim_type, dict(meta.optim_conf))
    rows_read, t_load = 0, time.time()

    for tid in sorted(meta.tables):
        t = meta.tables[tid]
        if t.table_type == C.TableType.kDense:
            value = None
            for d in shard_dirs.values():
                value = C.ckpt_load_dense(d, t.name)
                if value is not None:
                    break
            if value is None:
                raise C.KrakenError(f"no shard holds dense table {t.name!r}")
            new_id = engine.register_dense_table(t.name, value["val"], table_id=tid)
            engine.import_dense(new_id, t.name, value)
        else:
            new_id = engine.register_sparse_table(t.name, t.dimension, torch.float32, t.init_type, dict(t.init_conf),
                                                  table_id=tid)
            salt = engine._salt(new_id)
            if hasattr(engine, "import_sparse_routed"):
                # GPU shards: every rank reads 1 / world of the shard files (all their rows, multi-threaded) and
                # the rows are forwarded to their owners under the CURRENT placement on the device
                mine = [d for k, (_, d) in enumerate(sorted(shard_dirs.items())) if k % engine.world == engine.rank]
                rows_read += engine.import_sparse_routed(new_id, t.name, mine)
                continue
            for d in shard_dirs.values():
                cols = C.ckpt_load_sparse(d, t.name, 1, salt, engine.world, engine.rank)
                if cols is not None and cols["ids"].numel() > 0:
                    engine.import_sparse(new_id, cols)
    _barrier(engine)
    engine.last_checkpoint = {"op": "load", "rows_read": rows_read, "seconds": time.time() - t_load}
    return True
