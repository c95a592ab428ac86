"""Vectorised (numpy) versions of the 64-bit mixers of csrc/core/hash.h, for
host-side routing of id batches on the CPU backend."""
from __future__ import annotations

import numpy as np
import torch

_U = np.uint64


def mix64(v: np.ndarray) -> np.ndarray:
    """Bit-exact Mix64 over a uint64 array (wraps on overflow like the C++ code)."""
    with np.errstate(over="ignore"):
        v = v.astype(np.uint64, copy=True)
        v = v * _U(3935559000370003845) + _U(2691343689449507681)
        v ^= v >> _U(21)
        v ^= v << _U(37)
        v ^= v >> _U(4)
        v *= _U(4768777513237032717)
        v ^= v << _U(20)
        v ^= v >> _U(41)
        v ^= v << _U(5)
    return v


def owner_of(salt: int, ids: torch.Tensor, world: int) -> torch.Tensor:
    """Owner rank of every id (int64 tensor, reinterpreted as unsigned)."""
    a = ids.detach().cpu().contiguous().numpy().view(np.uint64)
    o = (mix64(a) ^ _U(salt)) % _U(world)
    return torch.from_numpy(o.astype(np.int64))
