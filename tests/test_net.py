"""Native TCP transport of the multi-process deployment (csrc/core/net.cc): the frame layout of the
reference's headers (kraken/rpc/protocol.h:12-41), a server that answers in the request's compression
(kraken/rpc/station.h:62-119) and a client whose calls time out (kraken/rpc/indep_connecter.h:83-84)."""
import socket
import struct
import threading
import time

import pytest

from kraken_b200._native import C


def echo_station(extra=None):
    calls = []

    def handler(rpc_type, body):
        calls.append((rpc_type, len(body)))
        if extra is not None:
            out = extra(rpc_type, body)
            if out is not None:
                return out
        return 0, bytes(body)[::-1]

    st = C.NetStation("127.0.0.1", 0, handler)
    st.start()
    return st, calls


def test_frame_bytes_are_the_reference_header_layout():
    """u32 body length, then the 13-byte header {u64 timestamp, u32 type | i32 error code, u8 compress}, then the
    body; a compressed body is a Snappy stream and the length counts the compressed bytes."""
    a, b = socket.socketpair()
    try:
        assert C.net_send_frame(a.fileno(), 0x0102030405060708, 24, b"hello", 0)
        raw = b.recv(64)
        assert raw == struct.pack("<IQiB", 5, 0x0102030405060708, 24, 0) + b"hello"
        assert C.net_send_frame(a.fileno(), 9, -1, b"", 0)
        assert b.recv(64) == struct.pack("<IQiB", 0, 9, -1, 0)
        body = b"abcd" * 4096
        assert C.net_send_frame(a.fileno(), 10, 3, body, 1)
        head = b.recv(17, socket.MSG_WAITALL)
        n, stamp, code, comp = struct.unpack("<IQiB", head)
        assert (stamp, code, comp) == (10, 3, 1) and n < len(body) // 10
        assert C.snappy_uncompress(b.recv(n, socket.MSG_WAITALL)) == body
        # and the other direction: frames assembled by hand are read back
        b.sendall(struct.pack("<IQiB", 3, 77, 5, 0) + b"xyz")
        assert C.net_recv_frame(a.fileno(), 1000) == (77, 5, b"xyz", 0)
        packed = C.snappy_compress(body)
        b.sendall(struct.pack("<IQiB", len(packed), 78, 0, 1) + packed)
        assert C.net_recv_frame(a.fileno(), 1000) == (78, 0, body, 1)
        assert C.net_recv_frame(a.fileno(), 50) == "timeout"
        b.sendall(struct.pack("<IQiB", 2, 79, 0, 7) + b"??")          # unknown compression code
        assert C.net_recv_frame(a.fileno(), 1000) == "bad frame"
        b.sendall(struct.pack("<IQiB", 100, 80, 0, 0) + b"short")     # the peer goes away in the middle of a frame
        b.close()
        assert C.net_recv_frame(a.fileno(), 1000) == "closed"
    finally:
        a.close()
        b.close()


def test_station_serves_many_clients_and_answers_in_the_requests_compression():
    st, calls = echo_station()
    try:
        errors = []

        def client(k):
            try:
                c = C.NetConnecter("127.0.0.1", st.port, 5000, k % 2)      # every other client compresses
                for i in range(40):
                    body = (b"%d-%d-" % (k, i)) * (1 + 300 * (i % 3))
                    assert c.call(100 + k, body, 0) == (0, 0, body[::-1])
                c.close()
            except Exception as e:   # surfaces in the main thread below
                errors.append(repr(e))

        threads = [threading.Thread(target=client, args=(k,)) for k in range(8)]
        [t.start() for t in threads]
        [t.join() for t in threads]
        assert not errors, errors
        assert len(calls) == 8 * 40 and {t for t, _ in calls} == set(range(100, 108))
        # a compressed request gets a compressed reply: look at the raw bytes
        raw = socket.create_connection(("127.0.0.1", st.port))
        assert C.net_send_frame(raw.fileno(), 1, 5, b"z" * 10_000, 1)
        n, stamp, code, comp = struct.unpack("<IQiB", raw.recv(17, socket.MSG_WAITALL))
        assert (stamp, code, comp) == (1, 0, 1) and n < 1000
        raw.close()
    finally:
        st.stop()


def test_timeouts_error_replies_and_late_replies():
    def behaviour(rpc_type, body):
        if rpc_type == 1:
            time.sleep(0.4)
        if rpc_type == 2:
            raise ValueError("handler failed")
        if rpc_type == 3:
            return 15, b"no such id"
        return None

    st, _ = echo_station(behaviour)
    try:
        c = C.NetConnecter("127.0.0.1", st.port, 5000, 0)
        t0 = time.perf_counter()
        status, _, msg = c.call(1, b"slow", 100)
        assert status == 17 and 0.08 < time.perf_counter() - t0 < 0.35 and b"no reply" in msg
        # the late reply to the call above arrives first and is dropped: this call gets its own reply
        assert c.call(0, b"abc", 2000) == (0, 0, b"cba")
        status, code, msg = c.call(2, b"", 0)
        assert (status, code) == (0, -1) and b"handler failed" in msg          # the server is still up
        assert c.call(3, b"", 0) == (0, 15, b"no such id")
        assert c.call(0, b"12", 0) == (0, 0, b"21")
        c.close()
        assert c.call(0, b"12", 0)[0] == 25                                      # kConnection: closed by us
    finally:
        st.stop()


def test_stop_ends_connections_and_a_lost_peer_is_reported():
    st, _ = echo_station()
    c = C.NetConnecter("127.0.0.1", st.port, 2000, 0)
    assert c.call(0, b"ab", 0) == (0, 0, b"ba")
    st.stop()
    st.stop()                                        # idempotent
    status, _, msg = c.call(0, b"ab", 500)
    assert status == 25, (status, msg)               # kConnection, not a hang until the timeout
    with pytest.raises(C.KrakenError):
        C.NetConnecter("127.0.0.1", st.port, 500, 0)  # nobody listens there any more


def test_message_bodies_pack_and_unpack_with_one_copy_per_tensor():
    """Body = u32 json_len | json | u32 n | n x (u64 len | tensor encoding).  The packer must write exactly what
    the per-tensor serializer writes (the format of kraken/common/serialize.h: layout byte, dims, dtype byte,
    payload), take non-contiguous and empty tensors, and the unpacker must reject truncated bodies."""
    import json

    import torch

    from kraken_b200.runtime import rpc
    ts = [torch.arange(12, dtype=torch.int64).view(3, 4), torch.randn(5, 8), torch.zeros(0, 4),
          torch.tensor([1, 2, 3], dtype=torch.int32), torch.randn(4, 6)[:, ::2], torch.randn(7).double()]
    meta = {"table_id": 3, "ids": [1, 2], "name": "x"}
    j = json.dumps(meta).encode()
    want = struct.pack("<I", len(j)) + j + struct.pack("<I", len(ts))
    for t in ts:
        b = C.serialize_tensor(t)
        want += struct.pack("<Q", len(b)) + b
    body = rpc.pack_body(meta, ts)
    assert body == want
    got_meta, got = rpc.unpack_body(body)
    assert got_meta == meta and len(got) == len(ts)
    for a, b in zip(ts, got):
        assert a.dtype == b.dtype and torch.equal(a, b)
    assert rpc.unpack_body(rpc.pack_body({}, [])) == ({}, [])
    # a tensor header that claims 2^40 x 2^20 floats in front of 8 bytes of payload must be refused before anything
    # of that size is allocated
    hdr = struct.pack("<BQqqB", 0, 2, 1 << 40, 1 << 20, 11)
    bomb = struct.pack("<I", 2) + b"{}" + struct.pack("<IQ", 1, len(hdr) + 8) + hdr + b"\0" * 8
    for bad in (body[:-1], body[:9], b"\x09\x00\x00\x00{}", body[:len(j) + 8] + b"\xff" * 8, bomb):
        with pytest.raises(C.KrakenError):
            rpc.unpack_body(bad)


def test_hostile_frames_do_not_take_the_server_down():
    """A length field that announces gigabytes, a Snappy header that claims an impossible expansion, an unknown
    compression code: the connection is dropped (or the frame refused), the station keeps serving others."""
    st, _ = echo_station()
    try:
        for bad in (struct.pack("<IQiB", 0xFFFFFFF0, 1, 0, 0) + b"tiny",                       # 4 GiB announced, 4 bytes sent
                    struct.pack("<IQiB", 6, 2, 0, 1) + b"\xff\xff\xff\xff\x0f\x00",             # Snappy: 4 GiB from 6 bytes
                    struct.pack("<IQiB", 3, 3, 0, 9) + b"abc"):                                 # compression code 9
            s = socket.create_connection(("127.0.0.1", st.port))
            s.sendall(bad)
            s.shutdown(socket.SHUT_WR)
            s.settimeout(5)
            try:
                assert s.recv(64) == b""        # no reply: the server closed the connection
            except ConnectionResetError:
                pass                            # ... with bytes of ours still unread
            s.close()
        c = C.NetConnecter("127.0.0.1", st.port, 2000, 1)
        assert c.call(7, b"still here", 0) == (0, 0, b"ereh llits")
        c.close()
    finally:
        st.stop()
    with pytest.raises(C.KrakenError):
        C.snappy_uncompress(b"\xff\xff\xff\xff\x0f\x00")      # claims 4 GiB, holds one byte
