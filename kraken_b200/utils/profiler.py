"""Per-step timing of the engine's phases and simple counters.

The reference has no tracing beyond a wall-clock print in one example
(examples/WideAndDeep/main.py:98-103).  Here every phase of a step (sparse pull,
sparse push, dense step, and whatever the user brackets with ``region``) is
timed on the device with CUDA events; the events of step t are read when step
t + 2 ends, so profiling never synchronises the host.  Set ``KRAKEN_PROFILE`` to
a file name to get one JSON line per step:

    {"step": 12, "rank": 0, "pull_ms": 0.21, "push_ms": 0.33, "dense_step_ms": 0.02, ...}
"""
from __future__ import annotations

import contextlib
import json
import os
import time
from collections import defaultdict, deque
from typing import Deque, Dict, List, Optional, Tuple

import torch


class StepProfiler:
    def __init__(self, path: Optional[str] = None, rank: int = 0, lag: int = 2) -> None:
        self.path = path
        self.rank = rank
        self.lag = lag
        self.cuda = torch.cuda.is_available()
        self.step = 0
        self._open: List[Tuple[str, object, object]] = []
        self._pending: Deque[Tuple[int, List[Tuple[str, object, object]], Dict[str, float]]] = deque()
        self.counters: Dict[str, float] = defaultdict(float)
        self.records: List[dict] = []
        self._fh = open(path, "a") if path else None

    @contextlib.contextmanager
    def region(self, name: str):
        if torch.cuda.is_available() and torch.cuda.is_current_stream_capturing():
            yield  # events inside a graph capture would be baked into the graph
            return
        if self.cuda:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            try:
                yield
            finally:
                e1.record()
                self._open.append((name, e0, e1))
        else:
            t0 = time.perf_counter()
            try:
                yield
            finally:
                self._open.append((name, t0, time.perf_counter()))

    def count(self, name: str, value: float = 1.0) -> None:
        self.counters[name] += value

    def end_step(self) -> None:
        self._pending.append((self.step, self._open, dict(self.counters)))
        self._open = []
        self.counters.clear()
        self.step += 1
        while len(self._pending) > self.lag:
            self._flush_one()

    def _flush_one(self) -> None:
        step, regions, counters = self._pending.popleft()
        rec: Dict[str, float] = {"step": step, "rank": self.rank}
        for name, a, b in regions:
            if self.cuda:
                b.synchronize()
                ms = a.elapsed_time(b)
            else:
                ms = (b - a) * 1e3
            rec[name + "_ms"] = rec.get(name + "_ms", 0.0) + ms
        rec.update(counters)
        self.records.append(rec)
        if self._fh:
            self._fh.write(json.dumps(rec) + "\n")
            self._fh.flush()

    def close(self) -> None:
        while self._pending:
            self._flush_one()
        if self._fh:
            self._fh.close()
            self._fh = None

    def summary(self) -> Dict[str, float]:
        """Mean of every timed phase over the recorded steps."""
        acc: Dict[str, List[float]] = defaultdict(list)
        for r in self.records:
            for k, v in r.items():
                if k.endswith("_ms"):
                    acc[k].append(v)
        return {k: sum(v) / len(v) for k, v in acc.items()}


def from_env(rank: int = 0) -> Optional[StepProfiler]:
    path = os.environ.get("KRAKEN_PROFILE")
    if not path:
        return None
    if rank:
        root, ext = os.path.splitext(path)
        path = f"{root}.rank{rank}{ext}"
    return StepProfiler(path, rank)


def engine_region(name: str):
    """Region of the process-global engine's profiler, or a no-op when profiling is off."""
    from ..pytorch import native
    if native.is_initialized():
        prof = getattr(native.engine(), "profiler", None)
        if prof is not None:
            return prof.region(name)
    return contextlib.nullcontext()
