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

Elastic scale-out (kraken/ps/ps.cc:336-477,553-602, kraken/scheduler/scheduler.cc:56-146): a
server may join while training runs.  The scheduler admits it only when every server reports
kWork, adds it to the ring (version + 1) and tells the older servers (kNotifyNodeJoin); each of
them moves the rows and dense tables that the new ring assigns to the newcomer (kTransfer*
messages, 65,536 rows per message, three attempts each), drops them, adopts the new ring and
answers.  Training never stops while rows move (the reference's proxy phase, kraken/ps/proxy.cc:29-145,
kraken/ps/ps_op.cc:10-127,141-164,315-357): every older server adopts the new ring at once, keeps serving
the rows it still owns and ships the others from a background thread; the newcomer serves from the first
moment in state kWork|kProxy - a request for a table or row it does not hold yet is answered after fetching
it on demand from the owner under the OLD ring (kTryFetch* messages, ids 15-18), and what a later transfer
message brings for a row that is already there is ignored (the copy that arrived first has since been
updated).  When the last older server reports kNotifyFinishTransfer the newcomer drops the proxy.  A worker
whose ring is stale gets kRouterVersion, refetches and re-partitions only the refused part of its request.
"""
from __future__ import annotations

import collections
import logging
import threading
from concurrent.futures import ThreadPoolExecutor
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
            # admission gate: nobody may be saving, loading or transferring (scheduler.cc:63-90)
            if self.clients and not self._all_working():
                return {"allow": False}, ()
            node_id = (max(self.nodes) + 1) if self.nodes else 0
            old_clients = dict(self.clients)
            meta_old_ring = _router_hex(self.router)
            self.router.add(node_id, meta["addr"])
            self.nodes[node_id] = meta["addr"]
            self.clients[node_id] = Connecter(meta["addr"])
            new = self.clients[node_id]
            rm = self._router_meta()
            old_ring_hex = meta_old_ring
            setup = dict(rm)
            if old_clients:
                # the newcomer serves at once, fetching what it lacks from the owners under the old ring
                setup.update({"proxy_old_router": old_ring_hex,
                              "proxy_nodes": {str(k): self.nodes[k] for k in old_clients},
                              "self_node": node_id})
            new.call(Rpc.FETCH_ROUTER, setup)
            if self.model is not None:
                new.call(Rpc.CREATE_MODEL, self.model)
                for t in self.tables.values():
                    if t["kind"] == "sparse":
                        new.call(Rpc.CREATE_SPARSE, t)
            # every older server adopts the ring and starts shipping what the new ring takes from it
            note = {**rm, "new_node": node_id, "new_addr": meta["addr"], "tables": list(self.tables.values())}
            notified = []
            try:
                for nid, c in old_clients.items():
                    c.call(Rpc.NOTIFY_NODE_JOIN, note, timeout_ms=60_000)
                    notified.append(nid)
            except Exception:
                # An older server could not be told: the newcomer is taken out of the ring again.  Servers that
                # had already adopted the new ring are given the old one back under a NEWER version, so workers
                # refetch; rows they have shipped meanwhile stay on the newcomer, which must be restarted to join.
                log.error("join of node %d failed after %d of %d servers had been notified", node_id, len(notified),
                          len(old_clients))
                self.router.remove(node_id)
                self.nodes.pop(node_id, None)
                self.clients.pop(node_id).close()
                back = self._router_meta()
                for c in old_clients.values():
                    try:
                        c.call(Rpc.FETCH_ROUTER, {**back, "cancel_transfer": True})
                    except Exception:
                        pass
                raise
            if old_clients:
                log.info("node %d joined: %d servers are shipping rows to it", node_id, len(old_clients))
            return {"allow": True, "node_id": node_id, **rm}, ()

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
        self.mu = threading.RLock()  # handlers run on one thread per connection: one at a time touches the shard
        self.rows_received = 0
        self.rows_fetched = 0          # rows this server pulled through the proxy while it was joining
        self.proxy: Optional[dict] = None   # while joining: {"ring", "vhash", "vnode", "peers": {node: Connecter}, "pending": set}
        self.tables_meta: Dict[int, dict] = {}
        self._transfer_thread: Optional[threading.Thread] = None
        self._cancel_transfer = False
        s = self.station
        s.register(Rpc.HEARTBEAT, lambda m, t: ({"status": self.status}, ()))
        for rpc, fn in ((Rpc.FETCH_ROUTER, self.set_router), (Rpc.CREATE_MODEL, self.create_model),
                        (Rpc.CREATE_DENSE, self.create_dense), (Rpc.CREATE_SPARSE, self.create_sparse),
                        (Rpc.PULL_DENSE, self.pull_dense), (Rpc.PUSH_DENSE, self.push_dense),
                        (Rpc.PULL_SPARSE, self.pull_sparse), (Rpc.PUSH_SPARSE, self.push_sparse),
                        (Rpc.COMBINE_PULL_DENSE, self.pull_dense), (Rpc.COMBINE_PULL_SPARSE, self.combine_pull_sparse),
                        (Rpc.COMBINE_PUSH_SPARSE, self.combine_push_sparse),
                        (Rpc.NOTIFY_SAVE, self.notify_save), (Rpc.NOTIFY_LOAD, self.notify_load),
                        (Rpc.NOTIFY_NODE_JOIN, self.notify_node_join), (Rpc.TRANSFER_DENSE, self.transfer_dense),
                        (Rpc.TRANSFER_SPARSE_VALUES, self.transfer_sparse_values),
                        (Rpc.TRANSFER_SPARSE_META, self.transfer_sparse_meta),
                        (Rpc.TRY_FETCH_DENSE, self.try_fetch_dense),
                        (Rpc.TRY_COMBINE_FETCH_DENSE, self.try_fetch_dense),
                        (Rpc.TRY_FETCH_SPARSE_META, self.try_fetch_sparse_meta),
                        (Rpc.TRY_FETCH_SPARSE_VALUES, self.try_fetch_sparse_values),
                        (Rpc.NOTIFY_FINISH_TRANSFER, self.notify_finish_transfer)):
            s.register(rpc, self._locked(fn))

    def _locked(self, fn):
        def run(meta, tensors):
            with self.mu:
                return fn(meta, tensors)
        return run

    def start(self, join_wait_s: float = 0.2, join_deadline_s: float = 120.0) -> None:
        """Registers with the scheduler.  While another server is saving, loading or transferring the
        scheduler answers "not now": retried with a x1.5 back-off (kraken/ps/ps.cc:396-422 sleeps 10 s)."""
        import time
        self.station.start()
        sched = Connecter(self.s_addr)
        wait, t0 = join_wait_s, time.monotonic()
        while True:
            meta, _ = sched.call(Rpc.TRY_JOIN, {"addr": self.addr}, timeout_ms=600_000)
            if meta.get("allow", True):
                break
            if time.monotonic() - t0 > join_deadline_s:
                raise RpcError(7, "the scheduler did not admit this server in time")
            time.sleep(wait)
            wait = min(wait * 1.5, 10.0)
        sched.close()
        with self.mu:
            self.node_id = meta["node_id"]
            self.set_router(meta, ())
            if self.proxy is None:
                self.status = C_STATUS_WORK  # first server, or every older server has already finished shipping
        log.info("ps %d joined at %s (ring version %d, %d rows received)", self.node_id, self.addr, self.version,
                 self.rows_received)

    def stop(self) -> None:
        self.station.stop()

    def _check(self, meta) -> None:
        # a server that ships rows away (kTransfer) or fetches them on demand (kProxy) keeps serving; one that is
        # saving, loading or not yet admitted does not (kraken/ps/ps_op.cc:129-139)
        if not (self.status & C_STATUS_WORK) or (self.status & (C_STATUS_SAVE | C_STATUS_LOAD)):
            raise RpcError(7)
        if meta.get("router_version", self.version) != self.version:
            raise RpcError(8)

    def set_router(self, meta, tensors):
        self.router = _router_from_hex(meta["router"])
        self.version = meta["version"]
        if meta.get("cancel_transfer"):
            self._cancel_transfer = True
        if "proxy_old_router" in meta:
            # this server has just been admitted next to older ones: serve at once, through the proxy
            ring = _router_from_hex(meta["proxy_old_router"])
            vn = ring.vnodes()
            self.node_id = int(meta["self_node"])
            self.proxy = {"ring": ring, "vhash": np.array([v[0] for v in vn], dtype=np.uint64),
                          "vnode": np.array([v[1] for v in vn], dtype=np.int64),
                          "peers": {int(k): Connecter(a, timeout_ms=60_000, compress=1)
                                    for k, a in meta["proxy_nodes"].items()},
                          "pending": {int(k) for k in meta["proxy_nodes"]}}
            self.status = C_STATUS_WORK | C_STATUS_PROXY
        return {}, ()

    # ---------------- proxy phase of a join (newcomer side): fetch on demand from the old owners
    def _proxy_owner(self, table_id: int, ids: torch.Tensor) -> np.ndarray:
        hv = mix64(ids.numpy().view(np.uint64)) ^ np.uint64(C.mix64(table_id))
        idx = np.searchsorted(self.proxy["vhash"], hv, side="left")
        idx[idx == len(self.proxy["vhash"])] = 0
        return self.proxy["vnode"][idx]

    def _proxy_sparse(self, table_id: int, ids: torch.Tensor) -> None:
        """Before a request touches ``ids``: rows this server does not hold yet are asked of their owners
        under the old ring and inserted if those had them (kraken/ps/ps_op.cc:315-357)."""
        if self.proxy is None or ids.numel() == 0:
            return
        if not self.shard.has_table(table_id):
            self._proxy_sparse_meta(table_id)
        ids = ids.reshape(-1).to(torch.int64).contiguous()
        missing = ids[self.shard.contains_sparse(table_id, ids) == 0]
        if missing.numel() == 0:
            return
        missing = torch.unique(missing)
        owners = self._proxy_owner(table_id, missing)
        for node in np.unique(owners):
            peer = self.proxy["peers"].get(int(node))
            if peer is None or int(node) not in self.proxy["pending"]:
                continue  # that owner has finished shipping: what it had for us is here already
            part = missing[torch.from_numpy(np.nonzero(owners == node)[0])]
            meta, ts = peer.call(Rpc.TRY_FETCH_SPARSE_VALUES, {"table_id": table_id}, [part])
            if ts and ts[0].numel() > 0:
                ns = len(meta["state_keys"])
                states = {int(k): x for k, x in zip(meta["state_keys"], ts[2:2 + ns])}
                states_i = {int(k): x for k, x in zip(meta["state_i_keys"], ts[2 + ns:])}
                self.shard.import_sparse(table_id, ts[0], ts[1], states, states_i, False)
                self.rows_fetched += int(ts[0].numel())

    def _proxy_sparse_meta(self, table_id: int) -> None:
        for peer in self.proxy["peers"].values():
            meta, _ = peer.call(Rpc.TRY_FETCH_SPARSE_META, {"table_id": table_id})
            if meta.get("exist"):
                self.create_sparse(meta["table"], ())
                return

    def _proxy_dense(self, table_ids: Sequence[int]) -> None:
        if self.proxy is None:
            return
        lacking = [int(t) for t in table_ids if not self.shard.has_table(int(t))]
        if not lacking:
            return
        by_owner: Dict[int, List[int]] = {}
        for t in lacking:
            by_owner.setdefault(int(self.proxy["ring"].hit(C.mix64(t))), []).append(t)
        for node, tids in by_owner.items():
            peer = self.proxy["peers"].get(node)
            if peer is None:
                continue
            meta, ts = peer.call(Rpc.TRY_COMBINE_FETCH_DENSE, {"table_ids": tids})
            pos = 0
            for ent in meta["exist"]:
                n = 1 + len(ent["state_keys"])
                self._import_dense(ent["table"], ent["state_keys"], ent["states_i"], ts[pos:pos + n])
                pos += n

    def create_model(self, meta, tensors):
        self.shard.init_model(meta["name"], C.OptimType(meta["optim_type"]), meta["optim_conf"])
        return {}, ()

    # ---------------- elastic scale-out: rows follow the ring to a server that has just joined
    def notify_node_join(self, meta, tensors):
        """Older server: adopt the new ring at once and ship, in the background, what it assigns to the
        newcomer.  Requests for rows this server keeps are served throughout; the rows to ship are frozen by the
        new ring itself (no worker on the new ring sends them here any more, one on the old ring is refused
        with kRouterVersion) and stay available to the newcomer's proxy until the shipment is complete."""
        new_ring = _router_from_hex(meta["router"])
        old_ring = self.router
        self.tables_meta = {int(t["id"]): t for t in meta["tables"]}
        self.router, self.version = new_ring, meta["version"]
        self.status = C_STATUS_WORK | C_STATUS_TRANSFER
        self._cancel_transfer = False
        self._transfer_thread = threading.Thread(target=self._transfer_to, daemon=True,
                                                 args=(meta, old_ring, new_ring, int(meta["new_node"])))
        self._transfer_thread.start()
        return {}, ()

    def _transfer_to(self, meta, old_ring, new_ring, new_node: int) -> None:
        """kraken/ps/ps.cc:336-372 (TransferTo): dense tables, then sparse rows in batches, then the rows that
        moved are dropped and the newcomer is told that this server has finished.  The shard lock is held only
        while a batch is copied out, never across a message to the newcomer."""
        moved = 0
        try:
            peer = Connecter(meta["new_addr"], timeout_ms=60_000, compress=1)  # server to server: compressed
            for t in meta["tables"]:
                tid = int(t["id"])
                if self._cancel_transfer:
                    return
                with self.mu:
                    if not self.shard.has_table(tid):
                        continue
                    if t["kind"] == "dense":
                        ship = old_ring.hit(C.mix64(tid)) == self.node_id and new_ring.hit(C.mix64(tid)) == new_node
                        v = self.shard.export_dense(tid) if ship else None
                    else:
                        cols = self.shard.export_sparse(tid)
                if t["kind"] == "dense":
                    if v is not None:
                        keys = sorted(int(k) for k in v["states"])
                        _send_with_retries(peer, Rpc.TRANSFER_DENSE,
                                           {"table": t, "state_keys": keys, "from": self.node_id,
                                            "states_i": {str(k): int(x) for k, x in v["states_i"].items()}},
                                           [v["val"]] + [v["states"][k] for k in keys])
                    continue
                _send_with_retries(peer, Rpc.TRANSFER_SPARSE_META, {"table": t, "from": self.node_id}, ())
                ids = cols["ids"]
                if ids.numel() == 0:
                    continue
                go = torch.from_numpy(np.nonzero(_ring_owners(new_ring, tid, ids) == new_node)[0])
                skeys = sorted(int(k) for k in cols["states"])
                ikeys = sorted(int(k) for k in cols["states_i"])
                for a in range(0, go.numel(), TRANSFER_ROWS):
                    if self._cancel_transfer:
                        return
                    sel = go[a:a + TRANSFER_ROWS]
                    _send_with_retries(peer, Rpc.TRANSFER_SPARSE_VALUES,
                                       {"table_id": tid, "state_keys": skeys, "state_i_keys": ikeys, "from": self.node_id},
                                       [ids[sel], cols["vals"][sel]] + [cols["states"][k][sel] for k in skeys]
                                       + [cols["states_i"][k][sel] for k in ikeys])
                moved += int(go.numel())
            # everything has arrived: what the new ring no longer assigns to this server is dropped
            # (kraken/ps/ps.cc:29-123), then the newcomer may stop asking this server
            with self.mu:
                for t in meta["tables"]:
                    if t["kind"] == "sparse" and self.shard.has_table(int(t["id"])):
                        self.shard.filter_sparse(int(t["id"]), 2, 0, 1, 0, new_ring, self.node_id)
            peer.call(Rpc.NOTIFY_FINISH_TRANSFER, {"from": self.node_id, "rows_moved": moved}, timeout_ms=60_000)
            peer.close()
            log.info("ps %d shipped %d rows to node %d", self.node_id, moved, new_node)
        except Exception as e:  # the rows stay here and stay reachable through the newcomer's proxy
            log.error("ps %d: transfer to node %d failed: %s", self.node_id, new_node, e)
        finally:
            with self.mu:
                self.status &= ~C_STATUS_TRANSFER

    def _import_dense(self, t: dict, state_keys, states_i, tensors) -> None:
        tid = int(t["id"])
        if self.shard.has_table(tid):
            return  # fetched through the proxy earlier: that copy has been updated since (ps.cc:745-750)
        self.shard.create_dense_table(tid, t["name"], tensors[0].view(*t["shape"]))
        v = {"val": tensors[0].view(*t["shape"]),
             "states": {int(k): x for k, x in zip(state_keys, tensors[1:])},
             "states_i": {int(k): int(x) for k, x in states_i.items()}}
        self.shard.import_dense(tid, t["name"], v)

    def transfer_dense(self, meta, tensors):
        self._import_dense(meta["table"], meta["state_keys"], meta["states_i"], tensors)
        return {}, ()

    def transfer_sparse_meta(self, meta, tensors):
        if not self.shard.has_table(int(meta["table"]["id"])):
            self.create_sparse(meta["table"], ())
        return {}, ()

    def transfer_sparse_values(self, meta, tensors):
        ns = len(meta["state_keys"])
        states = {int(k): x for k, x in zip(meta["state_keys"], tensors[2:2 + ns])}
        states_i = {int(k): x for k, x in zip(meta["state_i_keys"], tensors[2 + ns:])}
        # rows already here came through the proxy and may have been updated since: they win
        self.shard.import_sparse(int(meta["table_id"]), tensors[0], tensors[1], states, states_i, False)
        self.rows_received += int(tensors[0].numel())
        return {}, ()

    def notify_finish_transfer(self, meta, tensors):
        if self.proxy is not None and "from" in meta:
            self.proxy["pending"].discard(int(meta["from"]))
            if not self.proxy["pending"]:
                for c in self.proxy["peers"].values():
                    c.close()
                self.proxy = None
                self.status = C_STATUS_WORK
                log.info("ps %d: all transfers finished (%d rows received, %d fetched on demand)", self.node_id,
                         self.rows_received, self.rows_fetched)
        return {"rows_received": self.rows_received}, ()

    # ---------------- proxy phase (older server's side): hand out what the newcomer asks for
    def try_fetch_dense(self, meta, tensors):
        tids = meta["table_ids"] if "table_ids" in meta else [meta["table_id"]]
        exist, out = [], []
        for tid in tids:
            tid = int(tid)
            t = self.tables_meta.get(tid)
            if t is None or not self.shard.has_table(tid):
                continue
            v = self.shard.export_dense(tid)
            keys = sorted(int(k) for k in v["states"])
            exist.append({"table": t, "state_keys": keys, "states_i": {str(k): int(x) for k, x in v["states_i"].items()}})
            out += [v["val"]] + [v["states"][k] for k in keys]
        return {"exist": exist}, out

    def try_fetch_sparse_meta(self, meta, tensors):
        t = self.tables_meta.get(int(meta["table_id"]))
        return ({"exist": True, "table": t} if t is not None and t["kind"] == "sparse" else {"exist": False}), ()

    def try_fetch_sparse_values(self, meta, tensors):
        tid = int(meta["table_id"])
        if not self.shard.has_table(tid):
            return {"state_keys": [], "state_i_keys": []}, ()
        cols = self.shard.export_sparse_rows(tid, tensors[0].reshape(-1).to(torch.int64).contiguous())
        skeys = sorted(int(k) for k in cols["states"])
        ikeys = sorted(int(k) for k in cols["states_i"])
        return ({"state_keys": skeys, "state_i_keys": ikeys},
                [cols["ids"], cols["vals"]] + [cols["states"][k] for k in skeys] + [cols["states_i"][k] for k in ikeys])

    def create_dense(self, meta, tensors):
        self.shard.create_dense_table(meta["id"], meta["name"], tensors[0])
        return {}, ()

    def create_sparse(self, meta, tensors):
        self.shard.create_sparse_table(meta["id"], meta["name"], meta["dimension"],
                                       C.InitializerType(meta["init_type"]), meta["init_conf"])
        return {}, ()

    def pull_dense(self, meta, tensors):
        self._check(meta)
        self._proxy_dense(meta["table_ids"])
        return {}, [self.shard.pull_dense(t) for t in meta["table_ids"]]

    def push_dense(self, meta, tensors):
        self._check(meta)
        self._proxy_dense([meta["table_id"]])
        if meta.get("coo"):
            self.shard.push_dense_coo(meta["table_id"], tensors[0], tensors[1], meta["lr"])
        else:
            self.shard.push_dense(meta["table_id"], tensors[0], meta["lr"])
        return {}, ()

    def pull_sparse(self, meta, tensors):
        self._check(meta)
        self._proxy_sparse(meta["table_id"], tensors[0])
        return {}, [self.shard.pull_sparse(meta["table_id"], tensors[0])]

    def push_sparse(self, meta, tensors):
        self._check(meta)
        self._proxy_sparse(meta["table_id"], tensors[0])
        code = self.shard.push_sparse(meta["table_id"], tensors[0], tensors[1], meta["lr"])
        if code != 0:
            raise RpcError(code)
        return {}, ()

    def combine_pull_sparse(self, meta, tensors):
        """Several tables in one round trip (kraken/ps/ps_op.cc CombinePullSparseTable): ids of table k in tensor k."""
        self._check(meta)
        for t, ids in zip(meta["table_ids"], tensors):
            self._proxy_sparse(t, ids)
        return {}, [self.shard.pull_sparse(t, ids) for t, ids in zip(meta["table_ids"], tensors)]

    def combine_push_sparse(self, meta, tensors):
        """Tensors are (ids, summed gradients) pairs in the order of ``table_ids``."""
        self._check(meta)
        for k, t in enumerate(meta["table_ids"]):
            self._proxy_sparse(t, tensors[2 * k])
            code = self.shard.push_sparse(t, tensors[2 * k], tensors[2 * k + 1], meta["lr"])
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
                    if self.router.hit(C.mix64(t["id"])) != self.node_id:
                        continue  # moved to a server that joined later: the copy here is stale
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


# bit flags of kraken/common/info.h:26-37
C_STATUS_INIT, C_STATUS_WORK, C_STATUS_PROXY, C_STATUS_TRANSFER, C_STATUS_SAVE, C_STATUS_LOAD = 1, 2, 4, 8, 16, 32
TRANSFER_ROWS = 65536  # rows per kTransferSparseValues message (the reference sends 1024: kraken/ps/ps.cc:251)


def _ring_owners(router, table_id: int, ids: torch.Tensor) -> np.ndarray:
    """Node of every id on ``router``: ring.hit(Mix64(table_id) ^ Mix64(id)), vectorised."""
    vn = router.vnodes()
    vhash = np.array([v[0] for v in vn], dtype=np.uint64)
    vnode = np.array([v[1] for v in vn], dtype=np.int64)
    hv = mix64(ids.numpy().view(np.uint64)) ^ np.uint64(C.mix64(table_id))
    idx = np.searchsorted(vhash, hv, side="left")
    idx[idx == len(vhash)] = 0
    return vnode[idx]


def _send_with_retries(peer: "Connecter", rpc: int, meta: dict, tensors, attempts: int = 3):
    """A transfer message is tried three times before the join fails (kraken/ps/transfer.cc:37-47)."""
    for k in range(attempts):
        try:
            return peer.call(rpc, meta, tensors, timeout_ms=60_000)
        except RpcError as e:
            if k == attempts - 1 or e.code != 17:
                raise


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

    connecter_cls = Connecter    # how this worker reaches a scheduler or a server (a subclass may speak another wire)

    def __init__(self, cfg: EngineConfig, s_addr: str) -> None:
        super().__init__(cfg, 0, 1)
        self.device = torch.device("cpu")
        self.scheduler = self.connecter_cls(s_addr)   # control messages travel uncompressed, as in the reference
        self.compress = 1 if (cfg.compress is not None and int(getattr(cfg.compress, "value", cfg.compress)) != 0) else 0
        self.ps: Dict[int, Connecter] = {}
        self.dct_states: Dict[int, object] = {}
        self.refusals: Dict[int, int] = {}   # error code -> how often a server refused a request of this worker
        self._ring_lock = threading.RLock()
        self._refresh_router()
        # async_push: pushes are handed to one background thread (so they stay in order) and the caller goes on
        # with the next forward pass; a pull may then see rows from before the latest push - the reference's
        # fire-and-forget pushes (kraken/worker/emitter.cc:431-446, 539-549).  A push that failed raises at the
        # next push, pull or stop.
        self._pusher = ThreadPoolExecutor(max_workers=1, thread_name_prefix="kraken-push") if cfg.async_push else None
        self._push_futs: "collections.deque" = collections.deque()

    def _refresh_router(self) -> None:
        """Fetches the ring and publishes it as ONE tuple (router, version, vnode hashes, vnode owners): a request
        partitions its ids and stamps its version from the same tuple, whichever thread refreshes meanwhile
        (with ``async_push`` the push thread and the caller's thread both do)."""
        with self._ring_lock:
            meta, _ = self.scheduler.call(Rpc.FETCH_ROUTER)
            router = _router_from_hex(meta["router"])
            for nid, addr in meta["nodes"].items():
                if int(nid) not in self.ps:
                    self.ps[int(nid)] = self.connecter_cls(addr, compress=self.compress)
            vn = router.vnodes()
            vhash = np.array([v[0] for v in vn], dtype=np.uint64)
            vnode = np.array([v[1] for v in vn], dtype=np.int64)
            self._ring = (router, meta["version"], vhash, vnode,
                          torch.from_numpy(vhash.view(np.int64).copy()), torch.from_numpy(vnode.copy()))

    @property
    def router(self):
        return self._ring[0]

    @router.setter
    def router(self, r) -> None:   # the base class installs a placeholder ring before the first fetch
        old = getattr(self, "_ring", (None, 0, np.zeros(0, np.uint64), np.zeros(0, np.int64), None, None))
        self._ring = (r,) + tuple(old[1:])

    @property
    def version(self) -> int:
        return self._ring[1]

    @version.setter
    def version(self, v: int) -> None:   # tests age the ring with it
        r = self._ring
        self._ring = (r[0], int(v)) + tuple(r[2:])

    @staticmethod
    def _owners(ring, table_id: int, ids: torch.Tensor) -> np.ndarray:
        vhash, vnode = ring[2], ring[3]
        hv = mix64(ids.numpy().view(np.uint64)) ^ np.uint64(C.mix64(table_id))
        idx = np.searchsorted(vhash, hv, side="left")
        idx[idx == len(vhash)] = 0
        return vnode[idx]

    RETRY_CODES = (7, 8)  # kNodeStatus (server busy transferring / saving), kRouterVersion (our ring is old)

    def _backoff(self, attempt: int, code: int = 7) -> None:
        """After a refusal: count it (``refusals[code]``), wait if the server said it was busy, refetch the ring.
        A stale ring (8) needs no wait the first time: the scheduler already has the new one."""
        import time
        self.refusals[code] = self.refusals.get(code, 0) + 1
        if attempt >= 60:
            raise RpcError(7, "the servers stayed busy")
        if code != 8 or attempt > 0:
            time.sleep(min(0.02 * (1.5 ** attempt), 1.0))
        self._refresh_router()

    def _call_dense(self, table_id: int, rpc: int, meta: dict, tensors=()):
        """Calls the table's owner; if the server refuses (stale ring, or busy moving rows to a server
        that has just joined) the ring is refetched, the owner looked up again and the call repeated."""
        attempt = 0
        while True:
            router, version = self._ring[0], self._ring[1]
            owner = router.hit(C.mix64(table_id))
            try:
                return self.ps[owner].call(rpc, {**meta, "router_version": version}, tensors)
            except RpcError as e:
                if e.code not in self.RETRY_CODES:
                    raise
                self._backoff(attempt, e.code)
                attempt += 1

    def _call_sparse(self, rpc: int, table_id: int, meta: dict, ids: torch.Tensor, payload, done, attempt: int = 0):
        """Sends every id (with its payload row) to its owner.  A part that a server refuses is
        partitioned again on the refreshed ring and sent again, alone: parts that were accepted are
        never repeated, so a push is applied exactly once.  ``done(positions, reply_tensors)`` is called
        for every accepted part with the positions (into ``ids``) it covered."""
        # every part carries the version of the ring it was partitioned on: a refetch triggered by one refused part
        # (or by another thread) must not let the remaining parts of the OLD partition pass a server's version check
        ring = self._ring
        version = ring[1]
        nodes, order, counts = C.route_partition(ids, table_id, ring[4], ring[5])
        at = 0
        for node, cnt in zip(nodes, counts):
            # one server holds everything (a single-server deployment, or a small request): no index copies
            sel = None if len(nodes) == 1 else order[at:at + cnt]
            at += cnt
            part_ids = ids if sel is None else ids[sel]
            part_payload = None if payload is None else (payload if sel is None else payload[sel])
            try:
                _, ts = self.ps[int(node)].call(rpc, {**meta, "table_id": table_id, "router_version": version},
                                                [part_ids] + ([part_payload] if part_payload is not None else []))
            except RpcError as e:
                if e.code not in self.RETRY_CODES:
                    raise
                self._backoff(attempt, e.code)
                self._call_sparse(rpc, table_id, meta, part_ids, part_payload,
                                  (lambda pos, ts, sel=sel: done(pos if sel is None else sel[pos], ts)), attempt + 1)
                continue
            done(slice(None) if sel is None else sel, ts)

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
    def _submit_push(self, fn, *args) -> None:
        if self._pusher is None:
            fn(*args)
            return
        self._reap_pushes()
        self._push_futs.append(self._pusher.submit(fn, *args))

    def _reap_pushes(self, wait: bool = False) -> None:
        """Raises the error of a background push that has failed; ``wait``: blocks until every push is applied."""
        while self._push_futs and (wait or self._push_futs[0].done()):
            self._push_futs.popleft().result()

    def flush_pushes(self) -> None:
        """Returns when every push handed over so far has been applied on the servers."""
        self._reap_pushes(wait=True)

    def pull_dense_table(self, table_id):
        info = self._table(table_id, "dense")
        self._reap_pushes()
        _, ts = self._call_dense(table_id, Rpc.PULL_DENSE, {"table_ids": [table_id]})
        return ts[0].view(*info.shape)

    def push_dense_table(self, table_id, grad):
        self._table(table_id, "dense")
        g = grad.detach().to("cpu", torch.float32).contiguous().reshape(-1)
        st = self.dct_states.get(table_id)
        if st is not None:
            packed = C.cpu_dct_compress(g, self.cfg.life_span, self.cfg.eta, st)
            if packed is not None:
                self._submit_push(self._call_dense, table_id, Rpc.PUSH_DENSE,
                                  {"table_id": table_id, "lr": self.lr, "coo": True}, list(packed))
                return
        self._submit_push(self._call_dense, table_id, Rpc.PUSH_DENSE, {"table_id": table_id, "lr": self.lr}, [g])

    # sparse
    def pull_sparse_table(self, table_id, indices):
        info = self._table(table_id, "sparse")
        idx = indices.detach().to("cpu").to(torch.int64).contiguous()
        uniq, inv = C.cpu_dedup(idx.reshape(-1))
        parts = []
        self._reap_pushes()
        self._call_sparse(Rpc.PULL_SPARSE, table_id, {}, uniq, None, lambda pos, ts: parts.append((pos, ts[0])))
        if len(parts) == 1 and isinstance(parts[0][0], slice):
            rows = parts[0][1]            # one server answered for every id: its reply is the result
        else:
            rows = torch.empty((uniq.numel(), info.dimension), dtype=torch.float32)
            for pos, part in parts:
                rows[pos] = part
        return rows[inv].view(*idx.shape, info.dimension)

    def push_sparse_table(self, table_id, indices, grad):
        info = self._table(table_id, "sparse")
        idx = indices.detach().to("cpu").to(torch.int64).contiguous().reshape(-1)
        g = grad.detach().to("cpu", torch.float32).contiguous().view(-1, info.dimension)
        uniq, inv = C.cpu_dedup(idx)
        summed = C.cpu_segment_sum(g, inv, uniq.numel())
        self._submit_push(self._call_sparse, Rpc.PUSH_SPARSE, table_id, {"lr": self.lr}, uniq, summed,
                          lambda pos, ts: None)

    # several tables in one round trip per server (kCombinePull* / kCombinePushSparseTable of the reference)
    def combine_pull_dense_table(self, table_ids):
        by_owner: Dict[int, List[int]] = {}
        ring = self._ring
        for t in table_ids:
            self._table(t, "dense")
            by_owner.setdefault(ring[0].hit(C.mix64(t)), []).append(t)
        out: Dict[int, torch.Tensor] = {}
        version = ring[1]  # of the ring the owners above were looked up on
        for owner, tids in by_owner.items():
            try:
                _, ts = self.ps[owner].call(Rpc.COMBINE_PULL_DENSE, {"table_ids": tids, "router_version": version})
                for t, v in zip(tids, ts):
                    out[t] = v.view(*self.tables[t].shape)
            except RpcError as e:
                if e.code not in self.RETRY_CODES:
                    raise
                for t in tids:  # refused: table by table, each with its own retries on the refreshed ring
                    out[t] = self.pull_dense_table(t)
        return [out[t] for t in table_ids]

    def _combine_sparse(self, rpc: int, meta: dict, table_ids, uniqs, payloads, done) -> None:
        """One message per server carrying that server's part of every table.  A server that refuses
        gets its parts again table by table through ``_call_sparse`` (which re-partitions and retries)."""
        ring = self._ring
        owners = [self._owners(ring, t, u) for t, u in zip(table_ids, uniqs)]
        nodes = sorted({int(n) for o in owners for n in np.unique(o)})
        version = ring[1]  # of the ring this partition was made on (see _call_sparse)
        for node in nodes:
            sels = [torch.from_numpy(np.nonzero(o == node)[0]) for o in owners]
            ks = [k for k, sel in enumerate(sels) if sel.numel() > 0]
            tensors = []
            for k in ks:
                tensors.append(uniqs[k][sels[k]])
                if payloads is not None:
                    tensors.append(payloads[k][sels[k]])
            try:
                _, ts = self.ps[node].call(rpc, {**meta, "table_ids": [table_ids[k] for k in ks],
                                                 "router_version": version}, tensors)
                for j, k in enumerate(ks):
                    done(k, sels[k], [ts[j]] if ts else [])
            except RpcError as e:
                if e.code not in self.RETRY_CODES:
                    raise
                self._backoff(0, e.code)
                single = Rpc.PULL_SPARSE if payloads is None else Rpc.PUSH_SPARSE
                for k in ks:
                    self._call_sparse(single, table_ids[k], meta, uniqs[k][sels[k]],
                                      payloads[k][sels[k]] if payloads is not None else None,
                                      lambda pos, ts, k=k: done(k, sels[k][pos], ts), 1)

    def combine_pull_sparse_table(self, table_ids, indices):
        if len(table_ids) != len(indices):
            raise C.KrakenError("table_ids and indices differ in length")
        infos = [self._table(t, "sparse") for t in table_ids]
        idxs = [i.detach().to("cpu").to(torch.int64).contiguous() for i in indices]
        dd = [C.cpu_dedup(i.reshape(-1)) for i in idxs]
        rows = [torch.empty((u.numel(), info.dimension), dtype=torch.float32) for (u, _), info in zip(dd, infos)]

        def put(k, pos, ts):
            rows[k][pos] = ts[0]

        self._combine_sparse(Rpc.COMBINE_PULL_SPARSE, {}, list(table_ids), [u for u, _ in dd], None, put)
        return [r[inv].view(*i.shape, info.dimension) for r, (_, inv), i, info in zip(rows, dd, idxs, infos)]

    def combine_push_sparse_table(self, table_ids, indices, grads):
        if not (len(table_ids) == len(indices) == len(grads)):
            raise C.KrakenError("table_ids, indices and grads differ in length")
        uniqs, sums = [], []
        for t, i, g in zip(table_ids, indices, grads):
            info = self._table(t, "sparse")
            idx = i.detach().to("cpu").to(torch.int64).contiguous().reshape(-1)
            uniq, inv = C.cpu_dedup(idx)
            uniqs.append(uniq)
            sums.append(C.cpu_segment_sum(g.detach().to("cpu", torch.float32).contiguous().view(-1, info.dimension), inv,
                                          uniq.numel()))
        self._submit_push(self._combine_sparse, Rpc.COMBINE_PUSH_SPARSE, {"lr": self.lr}, list(table_ids), uniqs, sums,
                          lambda k, pos, ts: None)

    # checkpoints are written and read by the servers; the scheduler orchestrates
    def try_save_model(self) -> bool:
        self.flush_pushes()
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
        try:
            self.flush_pushes()
        finally:
            if self._pusher is not None:
                self._pusher.shutdown(wait=True)
            for c in list(self.ps.values()) + [self.scheduler]:
                c.close()
            super().stop()
