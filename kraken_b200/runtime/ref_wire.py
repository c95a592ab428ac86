"""The reference's binary serialisation (kraken/common/serialize.h, kraken/common/deserialize.h), as far as its
worker-facing messages need it: little-endian PODs, u64-counted vectors and strings, string maps, tensors
(dense, and the COO layout of its DCT emitter), the ring.  Shared by the ZeroMQ front end (requests in, replies
out) and the ZeroMQ client (the reverse)."""
from __future__ import annotations

import struct
from typing import Dict, List

import numpy as np
import torch

from .._native import C

# DType codes of the reference's tensors (kraken/t/element_type.h:23-37)
_DTYPES = {1: torch.bool, 2: torch.uint8, 3: torch.int8, 5: torch.int16, 7: torch.int32, 9: torch.int64,
           10: torch.float16, 11: torch.float32, 12: torch.float64}
_CODES = {v: k for k, v in _DTYPES.items()}
_UNSIGNED = {4: (np.uint16, torch.int32), 6: (np.uint32, torch.int64), 8: (np.uint64, torch.int64)}


class WireReader:
    """Cursor over a request body in the reference's serialisation (kraken/common/deserialize.h)."""

    def __init__(self, data: bytes) -> None:
        self.b, self.p = data, 0

    def _take(self, fmt: str):
        v = struct.unpack_from(fmt, self.b, self.p)
        self.p += struct.calcsize(fmt)
        return v[0]

    def u8(self): return self._take("<B")
    def u64(self): return self._take("<Q")
    def i64(self): return self._take("<q")
    def f32(self): return self._take("<f")
    def boolean(self): return self._take("<B") != 0

    def string(self) -> str:
        n = self.u64()
        s = self.b[self.p:self.p + n].decode()
        self.p += n
        return s

    def conf(self) -> Dict[str, str]:
        return {self.string(): self.string() for _ in range(self.u64())}

    def ids(self) -> torch.Tensor:
        n = self.u64()
        a = np.frombuffer(self.b, dtype=np.uint64, count=n, offset=self.p).view(np.int64).copy()
        self.p += 8 * n
        return torch.from_numpy(a)

    def u64_list(self) -> List[int]:
        return [int(x) for x in self.ids().numpy().view(np.uint64)]

    def tensor(self):
        """A dense tensor, or (indices, values, shape) for the COO layout the DCT emitter sends."""
        layout = self.u8()
        if layout == 1:
            idx, val = self.tensor(), self.tensor()
            return idx, val, [self.i64() for _ in range(self.u64())]
        dims = [self.i64() for _ in range(self.u64())]
        code = self.u8()
        numel = int(np.prod(dims)) if dims else 0          # a rank-0 shape has size 0 there (kraken/t/shape.cc:95-98)
        if code in _UNSIGNED:
            npdt, tdt = _UNSIGNED[code]
            a = np.frombuffer(self.b, dtype=npdt, count=numel, offset=self.p)
            self.p += a.nbytes
            return torch.from_numpy(a.astype(np.int64)).to(tdt).reshape(dims)
        dt = _DTYPES[code]
        nbytes = numel * torch.empty(0, dtype=dt).element_size()
        t = torch.frombuffer(bytearray(self.b[self.p:self.p + nbytes]), dtype=dt).reshape(dims) if numel else torch.empty(dims, dtype=dt)
        self.p += nbytes
        return t

    def rows(self) -> torch.Tensor:
        """vector<Tensor> of equally wide float32 vectors -> [n, dim]."""
        rows, self.p = C.wire_tensor_list_to_rows(self.b, self.p)
        return rows


def tensor_bytes(t: torch.Tensor) -> bytes:
    t = t.detach().contiguous()
    head = struct.pack("<BQ", 0, t.dim()) + b"".join(struct.pack("<q", d) for d in t.shape) + struct.pack("<B", _CODES[t.dtype])
    return head + t.numpy().tobytes()


def rewrite_ring(native: bytes, names: Dict[int, str]) -> bytes:
    """The deployment's ring (u64 version, nodes {u64 id, string name, vector<u64> vnodes}, virtual nodes
    {u64 hash, u64 node, string name}, kraken/common/serialize.h:350-395) with every node's name replaced."""
    r = WireReader(native)
    out = [struct.pack("<Q", r.u64())]
    n = r.u64()
    out.append(struct.pack("<Q", n))
    for _ in range(n):
        nid = r.u64()
        r.string()
        vn = r.ids()
        name = names[nid].encode()
        out.append(struct.pack("<QQ", nid, len(name)) + name + struct.pack("<Q", vn.numel()) + vn.numpy().tobytes())
    v = r.u64()
    out.append(struct.pack("<Q", v))
    for _ in range(v):
        h, nid = r.u64(), r.u64()
        old = r.string()
        name = (names[nid] + old[old.rfind("#"):] if "#" in old else names[nid]).encode()
        out.append(struct.pack("<QQQ", h, nid, len(name)) + name)
    return b"".join(out)
