"""Worker of this framework against servers of the REFERENCE: ``kk.initialize("zmq://host:port")``.

The counterpart of ``zmq_frontend.py``: a connecter that speaks the reference's wire protocol (a ZeroMQ DEALER
socket per peer, 13-byte header, its binary request and reply bodies, kraken/rpc/indep_connecter.cc:45-215 and
the ``*_prot.h`` files under kraken/protocol/) behind the ``call(rpc, meta, tensors)`` interface of this
package's own connecter, so that ``RemoteEngine`` - deduplication, routing over the ring, retries on a stale
ring, DCT compression, asynchronous pushes - runs unchanged against a Kraken cluster.  A job can so move its
workers first and its servers later.

What differs from the reference's own worker: every push waits for the server's (empty) reply unless
``async_push`` is set; requests have the reference's 5000 ms time limit (kraken/rpc/indep_connecter.h:83-84)
unless a call asks for more.
"""
from __future__ import annotations

import struct
import threading
import time
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .._native import C
from .engine import EngineConfig
from .remote import RemoteEngine
from .rpc import COMPRESS_NONE, Rpc, RpcError
from .ref_wire import WireReader, tensor_bytes

_F32 = 11   # DType code of float32 (kraken/t/element_type.h:23-37)


def _str(s: str) -> bytes:
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def _conf(c: Dict[str, str]) -> bytes:
    return struct.pack("<Q", len(c)) + b"".join(_str(str(k)) + _str(str(v)) for k, v in c.items())


def _ids(t: torch.Tensor) -> bytes:
    a = t.detach().to(torch.int64).contiguous().numpy()
    return struct.pack("<Q", a.size) + a.tobytes()


def _u64s(v: Sequence[int]) -> bytes:
    return struct.pack("<Q", len(v)) + b"".join(struct.pack("<Q", int(x)) for x in v)


def _coo(idx: torch.Tensor, val: torch.Tensor, numel: int) -> bytes:
    """A flat COO gradient as the reference's DCT emitter sends it: indices [1, nnz], values [nnz], shape [numel]."""
    return (struct.pack("<B", 1) + tensor_bytes(idx.to(torch.int64).reshape(1, -1)) + tensor_bytes(val.to(torch.float32).reshape(-1))
            + struct.pack("<Qq", 1, numel))


class ZmqConnecter:
    """``call(rpc, meta, tensors)`` of this package's connecter, carried out in the reference's wire format."""

    def __init__(self, addr: str, timeout_ms: int = 5000, compress: int = COMPRESS_NONE) -> None:
        import zmq
        self.zmq = zmq
        self.addr, self.compress, self.timeout_ms = addr, compress, timeout_ms
        self.ctx = zmq.Context.instance()
        self.sock = self.ctx.socket(zmq.DEALER)
        self.sock.setsockopt(zmq.LINGER, 0)
        self.sock.connect("tcp://" + addr)
        self.lock = threading.Lock()
        self.stamp = int(time.time() * 1e6)
        self.numel: Dict[int, int] = {}     # dense table id -> element count (a COO gradient carries the dense shape)

    # ------------------------------------------------------------------ bodies
    def _request(self, rpc: int, meta: dict, ts: Sequence[torch.Tensor]) -> bytes:
        v = struct.pack("<Q", int(meta.get("router_version", 0)))
        if rpc == Rpc.INIT_MODEL:
            return _str(meta["name"]) + struct.pack("<B", int(meta["optim_type"])) + _conf(meta["optim_conf"])
        if rpc == Rpc.REGISTER_DENSE:
            return _str(meta["name"]) + tensor_bytes(ts[0])
        if rpc == Rpc.REGISTER_SPARSE:
            return (_str(meta["name"]) + struct.pack("<qBB", int(meta["dimension"]), _F32, int(meta["init_type"]))
                    + _conf(meta["init_conf"]))
        if rpc in (Rpc.FETCH_ROUTER, Rpc.TRY_SAVE, Rpc.IS_ALL_PS_WORKING):
            return b""
        if rpc == Rpc.TRY_LOAD:
            return _str(meta["load_dir"])
        if rpc == Rpc.PULL_DENSE:
            return v + struct.pack("<Q", int(meta["table_ids"][0]))
        if rpc == Rpc.COMBINE_PULL_DENSE:
            return v + _u64s(meta["table_ids"])
        if rpc == Rpc.PUSH_DENSE:
            tid = int(meta["table_id"])
            grad = _coo(ts[0], ts[1], self.numel.get(tid, 0)) if meta.get("coo") else tensor_bytes(ts[0].to(torch.float32))
            return v + struct.pack("<Q", tid) + grad + struct.pack("<f", float(meta["lr"]))
        if rpc == Rpc.PULL_SPARSE:
            return v + struct.pack("<Q", int(meta["table_id"])) + _ids(ts[0])
        if rpc == Rpc.COMBINE_PULL_SPARSE:
            return v + struct.pack("<Q", len(ts)) + b"".join(struct.pack("<Q", int(t)) + _ids(i)
                                                              for t, i in zip(meta["table_ids"], ts))
        if rpc == Rpc.PUSH_SPARSE:
            return (v + struct.pack("<Q", int(meta["table_id"])) + _ids(ts[0]) + C.wire_rows_to_tensor_list(ts[1].to(torch.float32))
                    + struct.pack("<f", float(meta["lr"])))
        if rpc == Rpc.COMBINE_PUSH_SPARSE:
            tids = meta["table_ids"]
            items = b"".join(struct.pack("<Q", int(t)) + _ids(ts[2 * k]) + C.wire_rows_to_tensor_list(ts[2 * k + 1].to(torch.float32))
                             for k, t in enumerate(tids))
            return v + struct.pack("<Q", len(tids)) + items + struct.pack("<f", float(meta["lr"]))
        raise RpcError(1, f"type {rpc} has no counterpart in the reference's worker protocol")

    def _reply(self, rpc: int, meta: dict, body: bytes) -> Tuple[dict, List[torch.Tensor]]:
        r = WireReader(body)
        if rpc in (Rpc.REGISTER_DENSE, Rpc.REGISTER_SPARSE):
            return {"table_id": r.u64()}, []
        if rpc == Rpc.FETCH_ROUTER:
            ring = C.Router.from_bytes(body)
            nodes = {str(n): ring.node_name(n) for n in ring.node_ids()}
            return {"router": body.hex(), "nodes": nodes, "version": ring.version()}, []
        if rpc in (Rpc.TRY_SAVE, Rpc.TRY_LOAD):
            return {"success": r.boolean()}, []
        if rpc == Rpc.IS_ALL_PS_WORKING:
            return {"yes": r.boolean()}, []
        if rpc == Rpc.PULL_DENSE:
            return {}, [r.tensor().to(torch.float32).reshape(-1)]
        if rpc == Rpc.COMBINE_PULL_DENSE:
            return {}, [r.tensor().to(torch.float32).reshape(-1) for _ in range(r.u64())]
        if rpc == Rpc.PULL_SPARSE:
            return {}, [r.rows()]
        if rpc == Rpc.COMBINE_PULL_SPARSE:
            got = {}
            for _ in range(r.u64()):
                t = r.u64()
                got[t] = r.rows()
            return {}, [got[int(t)] for t in meta["table_ids"]]
        return {}, []

    # ------------------------------------------------------------------ transport
    def call(self, rpc_type: int, meta: Optional[dict] = None, tensors: Sequence[torch.Tensor] = (),
             timeout_ms: Optional[int] = None):
        meta = meta or {}
        rpc = int(rpc_type)
        body = self._request(rpc, meta, tensors)
        if self.compress == 1 and body:
            body = C.snappy_compress(body)
        limit = (timeout_ms or self.timeout_ms) / 1000.0
        with self.lock:
            self.stamp += 1
            stamp = self.stamp
            self.sock.send(struct.pack("<QIB", stamp, rpc, self.compress if body else 0) + body)
            deadline = time.monotonic() + limit
            while True:
                left = deadline - time.monotonic()
                if left <= 0 or not self.sock.poll(int(left * 1000) + 1):
                    raise RpcError(17, f"{self.addr} type {rpc}")
                msg = self.sock.recv()
                got, code, comp = struct.unpack_from("<QiB", msg, 0)
                if got == stamp:
                    break       # replies to calls that timed out earlier are dropped
        if code != 0:
            raise RpcError(code, f"{self.addr} type {rpc}")
        raw = msg[13:]
        if comp == 1 and raw:
            raw = C.snappy_uncompress(raw)
        return self._reply(rpc, meta, raw)

    def close(self) -> None:
        self.sock.close(linger=0)


class ZmqRemoteEngine(RemoteEngine):
    """``RemoteEngine`` over the reference's wire protocol: this framework's worker on a Kraken cluster."""

    connecter_cls = ZmqConnecter

    def __init__(self, cfg: EngineConfig, s_addr: str) -> None:
        if cfg.compress is None:
            cfg.compress = 1      # the reference's workers compress what they send to the servers (kraken/worker/emitter.cc:29)
        super().__init__(cfg, s_addr)

    def register_dense_table(self, name, val, table_id=None):
        tid = super().register_dense_table(name, val, table_id)
        for c in self.ps.values():
            c.numel[tid] = int(val.numel())
        self._numel = getattr(self, "_numel", {})
        self._numel[tid] = int(val.numel())
        return tid

    def _refresh_router(self) -> None:
        super()._refresh_router()
        for c in self.ps.values():          # connecters made for servers that joined since
            c.numel.update(getattr(self, "_numel", {}))
