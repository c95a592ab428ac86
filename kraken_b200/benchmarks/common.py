"""Shared helpers of the benchmark scripts: rank set-up, device timing (max over ranks), JSON output."""
from __future__ import annotations

import json
import os
import time

import torch
import torch.distributed as dist


def world_rank():
    return int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))


def sync_all():
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()
        if torch.cuda.is_available():
            torch.cuda.synchronize()


def max_over_ranks(value: float, device="cpu") -> float:
    if not (dist.is_initialized() and dist.get_world_size() > 1):
        return value
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


class DeviceTimer:
    """CUDA-event timer on the current stream (wall clock on CPU-only runs)."""

    def __init__(self):
        self.cuda = torch.cuda.is_available()
        if self.cuda:
            self.e0, self.e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def start(self):
        sync_all()
        if self.cuda:
            self.e0.record()
        self.t0 = time.perf_counter()

    def stop_ms(self) -> float:
        if self.cuda:
            self.e1.record()
            sync_all()
            ms = self.e0.elapsed_time(self.e1)
            dev = torch.device("cuda", torch.cuda.current_device())
        else:
            ms = (time.perf_counter() - self.t0) * 1e3
            dev = "cpu"
        return max_over_ranks(ms, dev)


def emit(record: dict) -> None:
    world, rank = world_rank()
    if rank == 0:
        print(json.dumps(record), flush=True)
