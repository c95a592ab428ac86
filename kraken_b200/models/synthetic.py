"""Synthetic click-through data of the shapes the benchmarks name: log1p of
LogNormal dense features, Zipf-distributed categorical ids, labels from a fixed
random teacher.  Everything is generated on the host (optionally into pinned
memory) so that a benchmark can include the host-to-device copy."""
from __future__ import annotations

from typing import Optional, Tuple

import numpy as np
import torch

from ..utils.hashing import mix64


def zipf_ids(rng: np.random.Generator, shape, vocab: int, s: float) -> np.ndarray:
    """Ranks in [0, vocab) with P(r) ~ (r + 1)^-s (inverse CDF of the continuous envelope)."""
    u = rng.random(shape)
    if abs(s - 1.0) < 1e-9:
        r = np.exp(u * np.log(vocab + 1.0)) - 1.0
    else:
        a = 1.0 - s
        r = ((float(vocab + 1) ** a - 1.0) * u + 1.0) ** (1.0 / a) - 1.0
    return np.minimum(r.astype(np.int64), vocab - 1)


class ClickDataset:
    """Batches of (dense [B, num_dense] f32, ids [B, F] i64 global ids, labels [B] f32)."""

    def __init__(self, num_fields: int = 26, num_dense: int = 13, vocab: int = 10_000_000, zipf_s: float = 1.1,
                 seed: int = 0, id_space: Optional[int] = None):
        self.F, self.D, self.vocab, self.s = num_fields, num_dense, int(vocab), float(zipf_s)
        self.id_space = id_space
        self.rng = np.random.default_rng(seed)
        t = np.random.default_rng(12345)
        self.w_dense = t.normal(0.0, 0.1, num_dense).astype(np.float32)
        self.w_field = t.normal(0.0, 0.1, num_fields).astype(np.float32)

    def batch(self, batch_size: int, pin: bool = False) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        B, F = batch_size, self.F
        dense = np.log1p(self.rng.lognormal(0.0, 1.0, (B, self.D))).astype(np.float32)
        local = zipf_ids(self.rng, (B, F), self.vocab, self.s)
        ids = local + (np.arange(F, dtype=np.int64) * self.vocab)[None, :]
        if self.id_space is not None:
            ids = (mix64(ids.reshape(-1).view(np.uint64)) % np.uint64(self.id_space)).astype(np.int64).reshape(B, F)
        # teacher: a pseudo-random feature in [-1, 1) per (field, id)
        h = (mix64(ids.reshape(-1).view(np.uint64)) >> np.uint64(40)).astype(np.float32).reshape(B, F)
        h = h / float(1 << 23) - 1.0
        logit = dense @ self.w_dense + h @ self.w_field
        labels = (self.rng.random(B) < 1.0 / (1.0 + np.exp(-logit))).astype(np.float32)
        out = (torch.from_numpy(dense), torch.from_numpy(ids), torch.from_numpy(labels))
        return tuple(t.pin_memory() for t in out) if pin else out


class MultiHotDataset:
    """Batches for the multi-hot model: dense [B, num_dense], one JaggedTensor of B * F bags
    (sample-major, field-minor) over a 2^40 hashed id space, labels [B]."""

    def __init__(self, num_fields: int = 100, num_dense: int = 13, vocab: int = 1_000_000, zipf_s: float = 1.1,
                 mean_len: float = 20.0, max_len: int = 100, id_bits: int = 40, seed: int = 0):
        self.F, self.D, self.vocab, self.s = num_fields, num_dense, int(vocab), float(zipf_s)
        self.mean_len, self.max_len, self.id_bits = mean_len, max_len, id_bits
        self.rng = np.random.default_rng(seed)
        self.w_dense = np.random.default_rng(54321).normal(0.0, 0.1, num_dense).astype(np.float32)

    def batch(self, batch_size: int, pin: bool = False):
        B, F = batch_size, self.F
        dense = np.log1p(self.rng.lognormal(0.0, 1.0, (B, self.D))).astype(np.float32)
        lens = np.clip(self.rng.poisson(self.mean_len, B * F), 1, self.max_len).astype(np.int64)
        offsets = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
        total = int(offsets[-1])
        field = np.repeat(np.tile(np.arange(F, dtype=np.int64), B), lens)
        local = zipf_ids(self.rng, total, self.vocab, self.s)
        ids = (mix64((local + field * self.vocab).view(np.uint64)) & np.uint64((1 << self.id_bits) - 1)).astype(np.int64)
        logit = dense @ self.w_dense
        labels = (self.rng.random(B) < 1.0 / (1.0 + np.exp(-logit))).astype(np.float32)
        out = [torch.from_numpy(dense), torch.from_numpy(ids), torch.from_numpy(offsets), torch.from_numpy(labels)]
        return [t.pin_memory() for t in out] if pin else out


def mnist_like(rng: np.random.Generator, means: np.ndarray, batch_size: int):
    """Images = class mean + N(0, 1) noise over 784 pixels, labels uniform over the classes."""
    y = rng.integers(0, means.shape[0], batch_size)
    x = means[y] + rng.normal(0.0, 1.0, (batch_size, means.shape[1])).astype(np.float32)
    return torch.from_numpy(x.astype(np.float32)), torch.from_numpy(y.astype(np.int64))
