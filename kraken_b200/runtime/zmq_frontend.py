"""ZeroMQ front end: workers of the REFERENCE train against a deployment of this framework.

The reference's worker library talks ZeroMQ (DEALER sockets) with a 13-byte header and hand-rolled binary
bodies (kraken/rpc/protocol.h:12-41, kraken/rpc/indep_connecter.cc:45-215, one ``*_prot.h`` per RPC under
kraken/protocol/).  This module listens the way its servers do - a ROUTER socket for the scheduler and one per
parameter server (kraken/rpc/station.cc:127-228) - decodes the worker-facing requests, forwards them to the
native ``scheduler_server`` / ``ps_server`` of this package over their own TCP transport and encodes the
replies.  A job can so move over in steps: first the servers, later the workers.

Covered: everything a worker sends (kraken/worker/emitter.cc): InitModel, RegisterDenseTable, RegisterSparseTable,
FetchRouter, TrySaveModel, TryLoadModel, IsAllPsWorking to the scheduler; PullDenseTable, CombinePullDenseTable,
PushDenseTable (dense or DCT-compressed COO), PullSparseTable, CombinePullSparseTable, PushSparseTable,
CombinePushSparseTable to the servers; Snappy bodies; error codes in the reply header (a stale ring is answered
with kRouterVersionError, after which the reference's worker refetches the ring, kraken/worker/emitter.cc:32-62).
Not covered: the server-to-server messages of the reference (join, transfer, proxy): its servers and these do
not mix.

The ring a worker receives is the deployment's own ring with the node names replaced by this front end's ZeroMQ
endpoints: a worker places ids with the virtual-node hashes it is given (kraken/common/router.cc:262-277) and
connects to the node names, so placement agrees with the native servers' ownership checks.

    python -m kraken_b200.runtime.zmq_frontend --s_addr 127.0.0.1:50000 --port 60000
"""
from __future__ import annotations

import argparse
import logging
import struct
import threading
from typing import Dict, List, Optional

import numpy as np
import torch

from .._native import C
from .ref_wire import WireReader, rewrite_ring, tensor_bytes
from .rpc import Connecter, Rpc, RpcError

log = logging.getLogger("kraken_b200")


class ZmqFrontend:
    def __init__(self, s_addr: str, host: str = "127.0.0.1", port: int = 0) -> None:
        import zmq
        self.zmq = zmq
        self.host = host
        self.ctx = zmq.Context()
        self.native_sched = Connecter(s_addr, timeout_ms=600_000)
        self.sched_sock = self.ctx.socket(zmq.ROUTER)
        self.port = self._bind(self.sched_sock, port)
        self.ps_socks: Dict[int, object] = {}       # node id -> ROUTER socket
        self.ps_addr: Dict[int, str] = {}            # node id -> "host:port" given to the workers
        self.ps_native: Dict[int, Connecter] = {}
        self.shapes: Dict[int, List[int]] = {}       # dense table id -> shape (replies carry it)
        self.stopping = False
        self.started = False
        self.threads: List[threading.Thread] = []     # one per ROUTER socket: requests to different servers run side by side
        self.lock = threading.Lock()
        self._discover()

    def _bind(self, sock, port: int) -> int:
        if port:
            sock.bind(f"tcp://{self.host}:{port}")
            return port
        return sock.bind_to_random_port(f"tcp://{self.host}")

    def _discover(self) -> dict:
        """A ROUTER socket and a native connection for every server of the deployment (new ones as they join)."""
        meta, _ = self.native_sched.call(Rpc.FETCH_ROUTER)
        with self.lock:
            for nid, addr in meta["nodes"].items():
                nid = int(nid)
                if nid not in self.ps_socks:
                    sock = self.ctx.socket(self.zmq.ROUTER)
                    self.ps_addr[nid] = f"{self.host}:{self._bind(sock, 0)}"
                    self.ps_native[nid] = Connecter(addr, timeout_ms=60_000, compress=1)
                    self.ps_socks[nid] = sock
                    if self.started:
                        self._serve(sock, nid)
        return meta

    # ------------------------------------------------------------------ scheduler messages
    def _scheduler(self, rpc: int, r: WireReader) -> bytes:
        call = self.native_sched.call
        if rpc == Rpc.INIT_MODEL:
            name, optim, conf = r.string(), r.u8(), r.conf()
            call(Rpc.INIT_MODEL, {"name": name, "optim_type": optim, "optim_conf": conf})
            return b""
        if rpc == Rpc.REGISTER_DENSE:
            name, val = r.string(), r.tensor()
            meta, _ = call(Rpc.REGISTER_DENSE, {"name": name}, [val.to(torch.float32)])
            self.shapes[int(meta["table_id"])] = list(val.shape)
            return struct.pack("<Q", meta["table_id"])
        if rpc == Rpc.REGISTER_SPARSE:
            name, dim, _etype, init, conf = r.string(), r.i64(), r.u8(), r.u8(), r.conf()
            meta, _ = call(Rpc.REGISTER_SPARSE, {"name": name, "dimension": dim, "init_type": init, "init_conf": conf})
            return struct.pack("<Q", meta["table_id"])
        if rpc == Rpc.FETCH_ROUTER:
            meta = self._discover()
            return rewrite_ring(bytes.fromhex(meta["router"]), self.ps_addr)
        if rpc == Rpc.TRY_SAVE:
            return struct.pack("<B", 1 if call(Rpc.TRY_SAVE)[0]["success"] else 0)
        if rpc == Rpc.TRY_LOAD:
            ok = call(Rpc.TRY_LOAD, {"load_dir": r.string()})[0]["success"]
            return struct.pack("<B", 1 if ok else 0)
        if rpc == Rpc.IS_ALL_PS_WORKING:
            return struct.pack("<B", 1 if call(Rpc.IS_ALL_PS_WORKING)[0]["yes"] else 0)
        raise RpcError(1, f"type {rpc}")     # kUnRegisterFuncError

    # ------------------------------------------------------------------ server messages
    def _dense_shape(self, tid: int, flat: torch.Tensor) -> torch.Tensor:
        shape = self.shapes.get(tid)
        return flat.reshape(shape) if shape is not None and int(np.prod(shape)) == flat.numel() else flat

    def _server(self, node: int, rpc: int, r: WireReader) -> bytes:
        call = self.ps_native[node].call
        version = r.u64()
        if rpc == Rpc.PULL_DENSE:
            tid = r.u64()
            _, ts = call(Rpc.PULL_DENSE, {"table_ids": [tid], "router_version": version})
            return tensor_bytes(self._dense_shape(tid, ts[0]))
        if rpc == Rpc.COMBINE_PULL_DENSE:
            tids = r.u64_list()
            _, ts = call(Rpc.COMBINE_PULL_DENSE, {"table_ids": tids, "router_version": version})
            return struct.pack("<Q", len(ts)) + b"".join(tensor_bytes(self._dense_shape(t, v)) for t, v in zip(tids, ts))
        if rpc == Rpc.PUSH_DENSE:
            tid, grad, lr = r.u64(), r.tensor(), r.f32()
            if isinstance(grad, tuple):       # COO from the DCT emitter: indices [1, nnz] into the flat table, values [nnz]
                idx, val, _shape = grad
                call(Rpc.PUSH_DENSE, {"table_id": tid, "lr": lr, "coo": True, "router_version": version},
                     [idx.reshape(-1).to(torch.int64), val.reshape(-1).to(torch.float32)])
            else:
                call(Rpc.PUSH_DENSE, {"table_id": tid, "lr": lr, "router_version": version},
                     [grad.to(torch.float32).reshape(-1)])
            return b""
        if rpc == Rpc.PULL_SPARSE:
            tid, ids = r.u64(), r.ids()
            _, ts = call(Rpc.PULL_SPARSE, {"table_id": tid, "router_version": version}, [ids])
            return C.wire_rows_to_tensor_list(ts[0])
        if rpc == Rpc.COMBINE_PULL_SPARSE:
            req = [(r.u64(), r.ids()) for _ in range(r.u64())]
            _, ts = call(Rpc.COMBINE_PULL_SPARSE, {"table_ids": [t for t, _ in req], "router_version": version},
                         [i for _, i in req])
            return struct.pack("<Q", len(req)) + b"".join(struct.pack("<Q", t) + C.wire_rows_to_tensor_list(v)
                                                          for (t, _), v in zip(req, ts))
        if rpc == Rpc.PUSH_SPARSE:
            tid, ids, grads, lr = r.u64(), r.ids(), r.rows(), r.f32()
            call(Rpc.PUSH_SPARSE, {"table_id": tid, "lr": lr, "router_version": version}, [ids, grads])
            return b""
        if rpc == Rpc.COMBINE_PUSH_SPARSE:
            items = [(r.u64(), r.ids(), r.rows()) for _ in range(r.u64())]
            lr = r.f32()
            tensors = [x for _, ids, grads in items for x in (ids, grads)]
            call(Rpc.COMBINE_PUSH_SPARSE, {"table_ids": [t for t, _, _ in items], "lr": lr, "router_version": version},
                 tensors)
            return b""
        raise RpcError(1, f"type {rpc}")

    # ------------------------------------------------------------------ loop
    def _answer(self, sock, node: Optional[int]) -> None:
        frames = sock.recv_multipart()
        ident, msg = frames[0], frames[-1]
        stamp, rpc, comp = struct.unpack_from("<QIB", msg, 0)
        code, body = 0, b""
        try:
            raw = msg[13:]
            if comp == 1:
                raw = C.snappy_uncompress(raw)
            elif comp != 0:
                raise RpcError(6)
            body = self._scheduler(rpc, WireReader(raw)) if node is None else self._server(node, rpc, WireReader(raw))
            if comp == 1 and body:
                body = C.snappy_compress(body)
        except RpcError as e:
            code, body = e.code, b""
        except (struct.error, KeyError, IndexError, ValueError, C.KrakenError) as e:
            log.warning("front end: request of type %d could not be decoded: %r", rpc, e)
            code, body = 4, b""               # kDeserializeRequestError
        sock.send_multipart([ident, struct.pack("<QiB", stamp, code, comp if code == 0 and body else 0) + body])

    def _serve(self, sock, node: Optional[int]) -> None:
        """A thread that owns ``sock`` from here on: requests of one socket are answered in order (a worker's pull
        behind its push sees the push), different sockets do not wait for one another."""
        def loop():
            poller = self.zmq.Poller()
            poller.register(sock, self.zmq.POLLIN)
            while not self.stopping:
                if poller.poll(200):
                    self._answer(sock, node)
            sock.close(linger=0)

        t = threading.Thread(target=loop, name=f"kraken-zmq-frontend-{'scheduler' if node is None else node}", daemon=True)
        t.start()
        self.threads.append(t)

    def start(self) -> None:
        with self.lock:
            self.started = True
            self._serve(self.sched_sock, None)
            for nid, sock in self.ps_socks.items():
                self._serve(sock, nid)

    def stop(self) -> None:
        self.stopping = True
        for t in self.threads:
            t.join(timeout=10)
        if not self.started:
            for s in [self.sched_sock] + list(self.ps_socks.values()):
                s.close(linger=0)
        self.ctx.term()
        for c in [self.native_sched] + list(self.ps_native.values()):
            c.close()


def main(argv=None) -> None:
    p = argparse.ArgumentParser(description="ZeroMQ front end for workers of the reference")
    p.add_argument("--s_addr", required=True, help="host:port of this package's scheduler_server")
    p.add_argument("--host", default="127.0.0.1", help="address the reference's workers reach this process at")
    p.add_argument("--port", type=int, default=60000, help="port that plays the reference's scheduler")
    a = p.parse_args(argv)
    from ..utils.log import configure
    configure("info")
    f = ZmqFrontend(a.s_addr, a.host, a.port)
    f.start()
    log.info("ZeroMQ front end: scheduler endpoint %s:%d, servers %s", a.host, f.port, f.ps_addr)
    threading.Event().wait()


if __name__ == "__main__":
    main()
