"""Symmetric (peer-mapped) device memory for one box of NVLink-connected GPUs.

Every rank allocates an arena of the same size, exports it as a CUDA IPC
handle and maps the arenas of all peers; kernels then address "buffer X of
rank p" as ``base[p] + offset_of_X`` and move data with plain loads and stores
over NVLink / NVSwitch.  The handle exchange is the only host-side collective
and uses whatever ``torch.distributed`` group is current (NCCL or gloo).

This is the transport that replaces the reference's ZeroMQ connecters
(kraken/rpc/indep_connecter.cc, kraken/rpc/group_connecters.h) on the GPU path.
"""
from __future__ import annotations

from typing import Dict, List, Sequence, Tuple

import torch
import torch.distributed as dist

from .._native import C

_ALIGN = 256


class Layout:
    """Packs named buffers into one arena with 256-byte alignment."""

    def __init__(self) -> None:
        self.size = 0
        self.entries: Dict[str, Tuple[int, Tuple[int, ...], torch.dtype]] = {}

    def add(self, name: str, shape: Sequence[int], dtype: torch.dtype) -> int:
        n = 1
        for d in shape:
            n *= int(d)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        off = self.size
        self.entries[name] = (off, tuple(int(d) for d in shape), dtype)
        self.size = (off + nbytes + _ALIGN - 1) // _ALIGN * _ALIGN
        return off

    def offset(self, name: str) -> int:
        return self.entries[name][0]


class SymmetricArena:
    """One arena per rank, mapped into every rank of ``group``."""

    def __init__(self, layout: Layout, rank: int, world: int, group=None, alias_peers: bool = False) -> None:
        """alias_peers=True maps every "peer" to the local arena instead of exchanging
        handles: one GPU then runs the multi-rank kernels against peers that never
        answer (used to test the bounded device-side waits)."""
        self.layout = layout
        self.rank = rank
        self.world = world
        self.heap = C.SymHeap(max(layout.size, _ALIGN), rank, world, alias_peers)
        if world > 1 and not alias_peers:
            handles: List[bytes] = [b""] * world
            dist.all_gather_object(handles, self.heap.handle(), group=group)
            self.heap.open(handles)
            # Nobody may touch a peer arena before everyone has mapped everything.
            dist.barrier(group=group)

    def window(self, name: str) -> torch.Tensor:
        """The local copy of a named buffer as a tensor (a view; keep the arena alive)."""
        off, shape, dtype = self.layout.entries[name]
        return self.heap.window(off, list(shape), dtype)

    def close(self) -> None:
        self.heap.close()
