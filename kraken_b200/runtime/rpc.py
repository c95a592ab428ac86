"""Request / reply transport of the multi-process CPU deployment.

The reference's processes talk ZeroMQ with a 13-byte header and a hand-rolled
binary body (kraken/rpc/protocol.h:12-41, kraken/rpc/station.cc,
kraken/rpc/indep_connecter.cc).  This is the same idea on plain TCP sockets:

    frame   = u32 body_len | header | body
    header  = u64 timestamp (correlation id) | u32 type (request) or i32 error_code (reply) | u8 compress
    body    = u32 json_len | json metadata | tensors, each in the framework's binary tensor encoding

Bodies may be compressed (header byte ``compress``: 0 = none, 1 = compressed): the reference
compresses worker<->server and server<->server bodies with Snappy and never the header
(kraken/common/compress.h:18-91, kraken/rpc/station.h:62-119 answers with the request's type).
Code 1 is a Snappy stream here too, written and read by the framework's own codec
(csrc/core/snappy_codec.h: the public block format, no library); a server answers in the
compression of the request.

RPC type numbers are the reference's (kraken/protocol/rpc_func_type.h:8-38).
A ``Station`` serves registered handlers on a thread pool; a ``Connecter`` is a
client with a send lock, a timeout (5 s default, as in
kraken/rpc/indep_connecter.h:83-84) and synchronous ``call``.
"""
from __future__ import annotations

import json
import socket
import struct
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from .._native import C

class Rpc:
    HEARTBEAT = 0
    TRY_JOIN = 1
    NOTIFY_NODE_JOIN = 2
    INIT_MODEL = 3
    REGISTER_DENSE = 4
    REGISTER_SPARSE = 5
    CREATE_MODEL = 6
    CREATE_DENSE = 7
    CREATE_SPARSE = 8
    NOTIFY_FINISH_TRANSFER = 10
    FETCH_ROUTER = 11
    TRANSFER_DENSE = 12
    TRANSFER_SPARSE_META = 13
    TRANSFER_SPARSE_VALUES = 14
    TRY_FETCH_DENSE = 15
    TRY_COMBINE_FETCH_DENSE = 16
    TRY_FETCH_SPARSE_META = 17
    TRY_FETCH_SPARSE_VALUES = 18
    PULL_DENSE = 19
    COMBINE_PULL_DENSE = 20
    PUSH_DENSE = 21
    PULL_SPARSE = 22
    COMBINE_PULL_SPARSE = 23
    PUSH_SPARSE = 24
    COMBINE_PUSH_SPARSE = 25
    TRY_SAVE = 26
    TRY_LOAD = 27
    NOTIFY_SAVE = 28
    NOTIFY_LOAD = 29
    IS_ALL_PS_WORKING = 30


class RpcError(RuntimeError):
    def __init__(self, code: int, what: str = ""):
        super().__init__(f"rpc error {code}: {C.error_message(code)} {what}".strip())
        self.code = code


def pack_body(meta: dict, tensors: Sequence[torch.Tensor] = ()) -> bytes:
    """u32 json_len | json | u32 n | n x (u64 len | tensor in the framework's binary tensor encoding)."""
    return C.rpc_pack_body(json.dumps(meta).encode(), list(tensors))


def unpack_body(body: bytes) -> Tuple[dict, List[torch.Tensor]]:
    j, tensors = C.rpc_unpack_body(body)
    return json.loads(j), tensors


COMPRESS_NONE, COMPRESS_SNAPPY = 0, 1   # CompressType::kNo / kSnappy, kraken/rpc/protocol.h:7-10


def send_frame(sock: socket.socket, stamp: int, code: int, body: bytes, compress: int = COMPRESS_NONE) -> None:
    """One frame onto a connected socket (the native framing code, csrc/core/net.cc, on the socket's descriptor)."""
    if not C.net_send_frame(sock.fileno(), stamp, code, bytes(body), compress):
        raise ConnectionError("peer closed the connection")


def recv_frame(sock: socket.socket, timeout_ms: int = -1) -> Tuple[int, int, bytes, int]:
    """(correlation id, type or error code, body as sent by the application, compression used)."""
    got = C.net_recv_frame(sock.fileno(), timeout_ms)
    if isinstance(got, str):
        if got == "timeout":
            raise socket.timeout("no frame in time")
        raise ConnectionError(f"peer {got}")
    return got


Handler = Callable[[dict, List[torch.Tensor]], Tuple[dict, Sequence[torch.Tensor]]]


class Station:
    """Threaded TCP server dispatching frames to registered handlers.  Sockets, framing, body compression
    and the thread per connection are native (csrc/core/net.cc); a request's body is unpacked, handled and
    the reply packed here, on the connection's thread."""

    def __init__(self, port: int, host: str = "0.0.0.0") -> None:
        self.handlers: Dict[int, Handler] = {}
        self.native = C.NetStation(host, port, self._dispatch)
        self.port = self.native.port

    def _dispatch(self, rpc_type: int, body: bytes) -> Tuple[int, bytes]:
        fn = self.handlers.get(rpc_type)
        try:
            if fn is None:
                raise RpcError(1, f"type {rpc_type}")
            meta, tensors = unpack_body(body)
            out_meta, out_tensors = fn(meta, tensors)
            return 0, pack_body(out_meta, out_tensors)
        except RpcError as e:
            return e.code, pack_body({"what": str(e)})
        except C.KrakenError as e:
            return -1, pack_body({"what": str(e)})
        except Exception as e:  # a failing handler must not take the server down
            return -1, pack_body({"what": repr(e)})

    def register(self, rpc_type: int, fn: Handler) -> None:
        self.handlers[rpc_type] = fn

    def start(self) -> None:
        self.native.start()

    def stop(self) -> None:
        self.native.stop()


class Connecter:
    """Client for one peer (native socket code, csrc/core/net.cc).  ``call`` is synchronous and thread-safe; a
    reply that does not arrive within ``timeout_ms`` raises kTimeout (17), an error reply raises with the
    server's code, a lost connection raises ConnectionError."""

    def __init__(self, addr: str, timeout_ms: int = 5000, compress: int = COMPRESS_NONE) -> None:
        host, port = addr.rsplit(":", 1)
        self.addr = addr
        self.compress = compress
        try:
            self.native = C.NetConnecter(host, int(port), int(timeout_ms), int(compress))
        except C.KrakenError as e:
            raise ConnectionError(str(e)) from e

    def call(self, rpc_type: int, meta: Optional[dict] = None, tensors: Sequence[torch.Tensor] = (),
             timeout_ms: Optional[int] = None) -> Tuple[dict, List[torch.Tensor]]:
        transport, code, body = self.native.call(int(rpc_type), pack_body(meta or {}, tensors), int(timeout_ms or 0))
        if transport == 17:
            raise RpcError(17, f"{self.addr} type {rpc_type}")
        if transport != 0:
            raise ConnectionError(bytes(body).decode(errors="replace"))
        try:
            out_meta, out_tensors = unpack_body(body)
        except Exception:
            if code == 0:
                raise
            out_meta, out_tensors = {"what": bytes(body).decode(errors="replace")}, []   # an error raised below the handler
        if code != 0:
            raise RpcError(code, out_meta.get("what", ""))
        return out_meta, out_tensors

    def close(self) -> None:
        self.native.close()
