"""Multi-process CPU deployment: scheduler, parameter-server shards, workers.

The reference's process model kept for hosts without GPUs and for its
deployment shape (kraken/scheduler/scheduler.cc, kraken/ps/ps.cc,
kraken/worker/emitter.cc): one scheduler owns the membership ring and the
table registry, N parameter servers own the rows the consistent-hash ring
assigns to them, and any number of independent workers pull values and push
gradients.  Placement is the reference's: a sparse row lives on
``ring.hit(Mix64(table_id) ^ Mix64(id))``, a dense table on
``ring.hit(Mix64(table_id))``.  A worker whose ring is stale gets
kRouterVersion (8), refetches it and retries once (kraken/worker/emitter.cc:32-62).

A server that joins after rows exist receives no rows from the older servers
(no live migration): add servers before training, or save and load to reshard.
"""
from __future__ import annotations

import logging
import threading
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .._native import C
from ..utils.hashing import mix64
from .engine import Engine, EngineConfig, TableInfo
from .rpc import Connecter, Rpc, RpcError, Station

log = logging.getLogger("kraken_b200")


def _opt_name(t) -> int:
    return int(t.value) if hasattr(t, "value") else int(t)


def _router_hex(r) -> str:
    return r.to_bytes().hex()


def _router_from_hex(h: str):
    return C.Router.from_bytes(bytes.fromhex(h))


# ------------------------------------------------------------------ scheduler
class SchedulerServer:
    def __init__(self, port: int = 50000) -> None:
        self.station = Station(port)
        self.port = self.station.port
        self.mu = threading.Lock()
        self.router = C.Router()
        self.nodes: Dict[int, str] = {}
        self.clients: Dict[int, Connecter] = {}
        self.model: Optional[dict] = None
        self.tables: Dict[int, dict] = {}
        self.by_name: Dict[str, int] = {}
        s = self.station
        s.register(Rpc.TRY_JOIN, self.try_join)
        s.register(Rpc.FETCH_ROUTER, self.fetch_router)
        s.register(Rpc.INIT_MODEL, self.init_model)
        s.register(Rpc.REGISTER_DENSE, self.register_dense)
        s.register(Rpc.REGISTER_SPARSE, self.register_sparse)
        s.register(Rpc.TRY_SAVE, self.try_save)
        s.register(Rpc.TRY_LOAD, self.try_load)
        s.register(Rpc.IS_ALL_PS_WORKING, self.is_all_working)

    def start(self) -> None:
        self.station.start()

    def stop(self) -> None:
        self.station.stop()

    def _broadcast(self, rpc: int, meta: dict, tensors=()) -> None:
        for c in self.clients.values():
            c.call(rpc, meta, tensors, timeout_ms=600_000)

    def _router_meta(self) -> dict:
        return {"router": _router_hex(self.router), "nodes": {str(k): v for k, v in self.nodes.items()},
                "version": self.router.version()}

    def try_join(self, meta, tensors):
        with self.mu:
            node_id = (max(self.nodes) + 1) if self.nodes else 0
            self.router.add(node_id, meta["addr"])
            self.nodes[node_id] = meta["addr"]
            self.clients[node_id] = Connecter(meta["addr"])
            new = self.clients[node_id]
            if self.model is not None:
                new.call(Rpc.CREATE_MODEL, self.model)
                for t in self.tables.values():
                    if t["kind"] == "sparse":
                        new.call(Rpc.CREATE_SPARSE, t)
            rm = self._router_meta()
            for nid, c in self.clients.items():
                c.call(Rpc.FETCH_ROUTER, rm)  # tells every shard the new ring and its version
            return {"node_id": node_id, **rm}, ()

    def fetch_router(self, meta, tensors):
        with self.mu:
            return self._router_meta(), ()

    def init_model(self, meta, tensors):
        with self.mu:
            if self.model is None:
                self.model = {"name": meta["name"], "optim_type": meta["optim_type"], "optim_conf": meta["optim_conf"]}
                self._broadcast(Rpc.CREATE_MODEL, self.model)
            return {}, ()

    def register_dense(self, meta, tensors):
        with self.mu:
            if self.model is None:
                raise RpcError(10)
            name = meta["name"]
            if name in self.by_name:
                t = self.tables[self.by_name[name]]
                if t["kind"] != "dense" or list(t["shape"]) != list(tensors[0].shape):
                    raise RpcError(19, name)
                return {"table_id": t["id"]}, ()
            tid = len(self.tables)
            t = {"id": tid, "name": name, "kind": "dense", "shape": list(tensors[0].shape)}
            owner = self.router.hit(C.mix64(tid))
            self.clients[owner].call(Rpc.CREATE_DENSE, t, tensors)
            self.tables[tid] = t
            self.by_name[name] = tid
            return {"table_id": tid}, ()

    def register_sparse(self, meta, tensors):
        with self.mu:
            if self.model is None:
                raise RpcError(10)
            name = meta["name"]
            if name in self.by_name:
                t = self.tables[self.by_name[name]]
                if t["kind"] != "sparse" or t["dimension"] != meta["dimension"] or t["init_type"] != meta["init_type"]:
                    raise RpcError(20, name)
                return {"table_id": t["id"]}, ()
            tid = len(self.tables)
            t = {"id": tid, "name": name, "kind": "sparse", "dimension": meta["dimension"],
                 "init_type": meta["init_type"], "init_conf": meta["init_conf"]}
            self._broadcast(Rpc.CREATE_SPARSE, t)
            self.tables[tid] = t
            self.by_name[name] = tid
            return {"table_id": tid}, ()

    def _all_working(self) -> bool:
        try:
            return all(c.call(Rpc.HEARTBEAT)[0]["status"] == 2 for c in self.clients.values())
        except RpcError:
            return False

    def is_all_working(self, meta, tensors):
        with self.mu:
            return {"yes": self._all_working()}, ()

    def try_save(self, meta, tensors):
        with self.mu:
            if self.model is None or not self._all_working():
                return {"success": False}, ()
            payload = {"model": self.model, "tables": list(self.tables.values()), **self._router_meta()}
            self._broadcast(Rpc.NOTIFY_SAVE, payload)
            return {"success": True}, ()

    def try_load(self, meta, tensors):
        with self.mu:
            if self.model is not None:
                return {"success": True}, ()  # already initialised: nothing is loaded
            dirs = C.ckpt_latest_shard_dirs(meta["load_dir"])
            if not dirs:
                return {"success": False}, ()
            mm = C.ckpt_load_model(dirs[min(dirs)])
            self.model = {"name": mm.name, "optim_type": _opt_name(mm.optim_type), "optim_conf": dict(mm.optim_conf)}
            for tid in sorted(mm.tables):
                t = mm.tables[tid]
                if t.table_type == C.TableType.kDense:
                    self.tables[tid] = {"id": tid, "name": t.name, "kind": "dense", "shape": list(t.shape)}
                else:
                    self.tables[tid] = {"id": tid, "name": t.name, "kind": "sparse", "dimension": t.dimension,
                                        "init_type": _opt_name(t.init_type), "init_conf": dict(t.init_conf)}
                self.by_name[t.name] = tid
            payload = {"load_dir": meta["load_dir"], "model": self.model, "tables": list(self.tables.values()),
                       **self._router_meta()}
            self._broadcast(Rpc.NOTIFY_LOAD, payload)
            return {"success": True}, ()


# ------------------------------------------------------------------ parameter server
class PsServer:
    def __init__(self, port: int, addr: str, s_addr: str, saved_dir: str = "", max_save_count: int = 3,
                 seed: int = 0) -> None:
        self.station = Station(port)
        self.port = self.station.port
        self.addr = addr if addr else f"127.0.0.1:{self.port}"
        self.s_addr = s_addr
        self.saved_dir, self.max_save_count = saved_dir, max_save_count
        self.shard = C.CpuShard(seed)
        self.status = C_STATUS_INIT
        self.node_id = -1
        self.router = C.Router()
        self.version = 0
        s = self.station
        s.register(Rpc.HEARTBEAT, lambda m, t: ({"status": self.status}, ()))
        s.register(Rpc.FETCH_ROUTER, self.set_router)
        s.register(Rpc.CREATE_MODEL, self.create_model)
        s.register(Rpc.CREATE_DENSE, self.create_dense)
        s.register(Rpc.CREATE_SPARSE, self.create_sparse)
        s.register(Rpc.PULL_DENSE, self.pull_dense)
        s.register(Rpc.PUSH_DENSE, self.push_dense)
        s.register(Rpc.PULL_SPARSE, self.pull_sparse)
        s.register(Rpc.PUSH_SPARSE, self.push_sparse)
        s.register(Rpc.NOTIFY_SAVE, self.notify_save)
        s.register(Rpc.NOTIFY_LOAD, self.notify_load)

    def start(self) -> None:
        self.station.start()
        meta, _ = Connecter(self.s_addr).call(Rpc.TRY_JOIN, {"addr": self.addr}, timeout_ms=60_000)
        self.node_id = meta["node_id"]
        self.set_router(meta, ())
        self.status = C_STATUS_WORK
        log.info("ps %d joined at %s (ring version %d)", self.node_id, self.addr, self.version)

    def stop(self) -> None:
        self.station.stop()

    def _check(self, meta) -> None:
        if self.status != C_STATUS_WORK:
            raise RpcError(7)
        if meta.get("router_version", self.version) != self.version:
            raise RpcError(8)

    def set_router(self, meta, tensors):
        self.router = _router_from_hex(meta["router"])
        self.version = meta["version"]
        return {}, ()

    def create_model(self, meta, tensors):
        self.shard.init_model(meta["name"], C.OptimType(meta["optim_type"]), meta["optim_conf"])
        return {}, ()

    def create_dense(self, meta, tensors):
        self.shard.create_dense_table(meta["id"], meta["name"], tensors[0])
        return {}, ()

    def create_sparse(self, meta, tensors):
        self.shard.create_sparse_table(meta["id"], meta["name"], meta["dimension"],
                                       C.InitializerType(meta["init_type"]), meta["init_conf"])
        return {}, ()

    def pull_dense(self, meta, tensors):
        self._check(meta)
        return {}, [self.shard.pull_dense(t) for t in meta["table_ids"]]

    def push_dense(self, meta, tensors):
        self._check(meta)
        if meta.get("coo"):
            self.shard.push_dense_coo(meta["table_id"], tensors[0], tensors[1], meta["lr"])
        else:
            self.shard.push_dense(meta["table_id"], tensors[0], meta["lr"])
        return {}, ()

    def pull_sparse(self, meta, tensors):
        self._check(meta)
        return {}, [self.shard.pull_sparse(meta["table_id"], tensors[0])]

    def push_sparse(self, meta, tensors):
        self._check(meta)
        code = self.shard.push_sparse(meta["table_id"], tensors[0], tensors[1], meta["lr"])
        if code != 0:
            raise RpcError(code)
        return {}, ()

    def notify_save(self, meta, tensors):
        if not self.saved_dir:
            raise RpcError(23, "the server was started without --saved_dir")
        self.status |= C_STATUS_SAVE
        try:
            out = C.ckpt_prepare_save_dir(self.saved_dir, self.node_id, self.max_save_count)
            C.ckpt_save_router(out, _router_from_hex(meta["router"]))
            C.ckpt_save_model(out, self.shard.meta() if not meta["tables"] else _model_meta(meta))
            for t in meta["tables"]:
                if not self.shard.has_table(t["id"]):
                    continue
                if t["kind"] == "dense":
                    C.ckpt_save_dense(out, t["id"], t["name"], self.shard.export_dense(t["id"]))
                else:
                    cols = self.shard.export_sparse(t["id"])
                    C.ckpt_save_sparse(out, t["id"], t["name"], t["dimension"], C.InitializerType(t["init_type"]),
                                       t["init_conf"], cols["ids"], cols["vals"], cols["states"], cols["states_i"])
        finally:
            self.status &= ~C_STATUS_SAVE
        return {}, ()

    def notify_load(self, meta, tensors):
        self.status = C_STATUS_LOAD
        try:
            self.set_router(meta, ())
            self.create_model(meta["model"], ())
            dirs = C.ckpt_latest_shard_dirs(meta["load_dir"])
            for t in meta["tables"]:
                if t["kind"] == "dense":
                    if self.router.hit(C.mix64(t["id"])) != self.node_id:
                        continue
                    for d in dirs.values():
                        v = C.ckpt_load_dense(d, t["name"])
                        if v is not None:
                            self.shard.import_dense(t["id"], t["name"], v)
                            break
                else:
                    self.create_sparse(t, ())
                    for d in dirs.values():
                        cols = C.ckpt_load_sparse(d, t["name"], 2, 0, 1, 0, self.router, t["id"], self.node_id)
                        if cols is not None and cols["ids"].numel() > 0:
                            self.shard.import_sparse(t["id"], cols["ids"], cols["vals"], cols["states"], cols["states_i"])
        finally:
            self.status = C_STATUS_WORK
        return {}, ()


C_STATUS_INIT, C_STATUS_WORK, C_STATUS_SAVE, C_STATUS_LOAD = 1, 2, 16, 32


def _model_meta(meta: dict):
    m = C.ModelMeta()
    m.name = meta["model"]["name"]
    m.optim_type = C.OptimType(meta["model"]["optim_type"])
    m.optim_conf = meta["model"]["optim_conf"]
    tables = {}
    for t in meta["tables"]:
        tm = C.TableMeta()
        tm.id, tm.name = t["id"], t["name"]
        if t["kind"] == "dense":
            tm.table_type, tm.shape = C.TableType.kDense, t["shape"]
        else:
            tm.table_type, tm.dimension = C.TableType.kSparse, t["dimension"]
            tm.init_type, tm.init_conf = C.InitializerType(t["init_type"]), t["init_conf"]
        tables[t["id"]] = tm
    m.tables = tables
    return m


# ------------------------------------------------------------------ worker
class RemoteEngine(Engine):
    """Worker-side engine of the multi-process deployment (``initialize("host:port")``)."""

    def __init__(self, cfg: EngineConfig, s_addr: str) -> None:
        super().__init__(cfg, 0, 1)
        self.device = torch.device("cpu")
        self.scheduler = Connecter(s_addr)
        self.ps: Dict[int, Connecter] = {}
        self.dct_states: Dict[int, object] = {}
        self._refresh_router()

    def _refresh_router(self) -> None:
        meta, _ = self.scheduler.call(Rpc.FETCH_ROUTER)
        self.router = _router_from_hex(meta["router"])
        self.version = meta["version"]
        for nid, addr in meta["nodes"].items():
            if int(nid) not in self.ps:
                self.ps[int(nid)] = Connecter(addr)
        vn = self.router.vnodes()
        self._vhash = np.array([v[0] for v in vn], dtype=np.uint64)
        self._vnode = np.array([v[1] for v in vn], dtype=np.int64)

    def _owners(self, table_id: int, ids: torch.Tensor) -> np.ndarray:
        hv = mix64(ids.numpy().view(np.uint64)) ^ np.uint64(C.mix64(table_id))
        idx = np.searchsorted(self._vhash, hv, side="left")
        idx[idx == len(self._vhash)] = 0
        return self._vnode[idx]

    def _call_ps(self, node: int, rpc: int, meta: dict, tensors=()):
        """One retry after refetching the ring when the server says ours is stale."""
        try:
            return self.ps[node].call(rpc, {**meta, "router_version": self.version}, tensors)
        except RpcError as e:
            if e.code != 8:
                raise
            self._refresh_router()
            return self.ps[node].call(rpc, {**meta, "router_version": self.version}, tensors)

    # registry: the scheduler owns it
    def init_model(self, model_name, optim_type, optim_conf=None):
        self.scheduler.call(Rpc.INIT_MODEL, {"name": model_name, "optim_type": _opt_name(optim_type),
                                             "optim_conf": dict(optim_conf or {})})
        self.model_name, self.optim_type, self.optim_conf = model_name, optim_type, dict(optim_conf or {})

    def register_dense_table(self, name, val, table_id=None):
        v = val.detach().to("cpu", torch.float32).contiguous()
        meta, _ = self.scheduler.call(Rpc.REGISTER_DENSE, {"name": name}, [v])
        tid = meta["table_id"]
        self.tables[tid] = TableInfo(id=tid, name=name, kind="dense", shape=tuple(v.shape))
        self.name_to_id[name] = tid
        if self.cfg.emitter_type == C.EmitterType.kDCT:
            self.dct_states.setdefault(tid, C.DctState())
        return tid

    def register_sparse_table(self, name, dimension, dtype, init_type, init_conf, table_id=None):
        meta, _ = self.scheduler.call(Rpc.REGISTER_SPARSE, {"name": name, "dimension": int(dimension),
                                                            "init_type": _opt_name(init_type),
                                                            "init_conf": dict(init_conf)})
        tid = meta["table_id"]
        self.tables[tid] = TableInfo(id=tid, name=name, kind="sparse", dimension=int(dimension), init_type=init_type,
                                     init_conf=dict(init_conf))
        self.name_to_id[name] = tid
        self._refresh_router()
        return tid

    # dense
    def pull_dense_table(self, table_id):
        info = self._table(table_id, "dense")
        owner = self.router.hit(C.mix64(table_id))
        _, ts = self._call_ps(owner, Rpc.PULL_DENSE, {"table_ids": [table_id]})
        return ts[0].view(*info.shape)

    def push_dense_table(self, table_id, grad):
        self._table(table_id, "dense")
        g = grad.detach().to("cpu", torch.float32).contiguous().reshape(-1)
        owner = self.router.hit(C.mix64(table_id))
        st = self.dct_states.get(table_id)
        if st is not None:
            packed = C.cpu_dct_compress(g, self.cfg.life_span, self.cfg.eta, st)
            if packed is not None:
                self._call_ps(owner, Rpc.PUSH_DENSE, {"table_id": table_id, "lr": self.lr, "coo": True}, list(packed))
                return
        self._call_ps(owner, Rpc.PUSH_DENSE, {"table_id": table_id, "lr": self.lr}, [g])

    # sparse
    def pull_sparse_table(self, table_id, indices):
        info = self._table(table_id, "sparse")
        idx = indices.detach().to("cpu").to(torch.int64).contiguous()
        uniq, inv = C.cpu_dedup(idx.reshape(-1))
        owners = self._owners(table_id, uniq)
        rows = torch.empty((uniq.numel(), info.dimension), dtype=torch.float32)
        for node in np.unique(owners):
            sel = torch.from_numpy(np.nonzero(owners == node)[0])
            _, ts = self._call_ps(int(node), Rpc.PULL_SPARSE, {"table_id": table_id}, [uniq[sel]])
            rows[sel] = ts[0]
        return rows[inv].view(*idx.shape, info.dimension)

    def push_sparse_table(self, table_id, indices, grad):
        info = self._table(table_id, "sparse")
        idx = indices.detach().to("cpu").to(torch.int64).contiguous().reshape(-1)
        g = grad.detach().to("cpu", torch.float32).contiguous().view(-1, info.dimension)
        uniq, inv = C.cpu_dedup(idx)
        summed = C.cpu_segment_sum(g, inv, uniq.numel())
        owners = self._owners(table_id, uniq)
        for node in np.unique(owners):
            sel = torch.from_numpy(np.nonzero(owners == node)[0])
            self._call_ps(int(node), Rpc.PUSH_SPARSE, {"table_id": table_id, "lr": self.lr}, [uniq[sel], summed[sel]])

    # checkpoints are written and read by the servers; the scheduler orchestrates
    def try_save_model(self) -> bool:
        return bool(self.scheduler.call(Rpc.TRY_SAVE, timeout_ms=600_000)[0]["success"])

    def try_load_model_blocked(self, load_dir: str) -> bool:
        import time
        if not self.scheduler.call(Rpc.TRY_LOAD, {"load_dir": load_dir}, timeout_ms=600_000)[0]["success"]:
            return False
        wait = 0.05
        while not self.scheduler.call(Rpc.IS_ALL_PS_WORKING)[0]["yes"]:
            time.sleep(wait)
            wait = min(wait * 1.5, 5.0)
        self._refresh_router()
        return True

    def stop(self):
        for c in list(self.ps.values()) + [self.scheduler]:
            c.close()
        super().stop()
