"""Shared helpers of the benchmark scripts: rank set-up, device timing (max over ranks), JSON output."""
from __future__ import annotations

import json
import os
import time
from typing import Optional

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


def measure_copy_gbs(device=None, mib: int = 1024, reps: int = 5) -> float:
    """Device copy bandwidth in GB/s (read + write bytes of ``dst.copy_(src)`` over ``mib`` MiB, best of
    ``reps``, CUDA events): the denominator of the HBM side of a roofline, measured where the benchmark runs."""
    dev = device or torch.device("cuda", torch.cuda.current_device())
    n = mib << 20
    a, b = torch.empty(n, dtype=torch.uint8, device=dev), torch.empty(n, dtype=torch.uint8, device=dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    best = float("inf")
    for _ in range(reps + 1):
        e0.record()
        b.copy_(a)
        e1.record()
        torch.cuda.synchronize(dev)
        best = min(best, e0.elapsed_time(e1))
    return 2.0 * n / (best * 1e-3) / 1e9


def measure_peer_gbs(mib: int = 256, reps: int = 5) -> float:
    """Per-direction bandwidth in GB/s of a copy from this rank's GPU into the next rank's (every rank
    copies at the same time, so all links are busy as in an exchange); the minimum over ranks.  0 when there
    is one rank.  This is the link figure the NVLink side of a roofline divides by."""
    world, rank = world_rank()
    if world <= 1 or torch.cuda.device_count() < world:
        return 0.0
    me = torch.device("cuda", torch.cuda.current_device())
    peer = torch.device("cuda", (torch.cuda.current_device() + 1) % world)
    n = mib << 20
    src = torch.empty(n, dtype=torch.uint8, device=me)
    dst = torch.empty(n, dtype=torch.uint8, device=peer)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    best = float("inf")
    for _ in range(reps + 1):
        sync_all()
        e0.record()
        dst.copy_(src, non_blocking=True)
        e1.record()
        torch.cuda.synchronize(me)
        best = min(best, e0.elapsed_time(e1))
    gbs = n / (best * 1e-3) / 1e9
    t = torch.tensor([gbs], dtype=torch.float64, device=me)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    del src, dst
    return float(t.item())


class NvlinkCounters:
    """NVLink bytes sent and received by this rank's GPU, read from NVML's per-device throughput counters
    (fields NVLINK_THROUGHPUT_DATA_TX / RX; payload bytes, in KiB; asked for all links at once, else link by
    link).  Reading only: nothing on the GPU is configured.  ``read()`` returns (tx_bytes, rx_bytes) or None
    where the driver does not expose the counters (``why`` then says what failed); differences between two
    reads are the traffic in between."""

    def __init__(self, device: Optional[torch.device] = None) -> None:
        self.handle, self.why, self.per_link = None, "", False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            dev = torch.cuda.current_device() if device is None else (device.index or 0)
            uuid = getattr(torch.cuda.get_device_properties(dev), "uuid", None)
            try:
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + str(uuid)).encode())
            except Exception:
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(dev)
        except Exception as e:   # no NVML, or no such device in this container
            self.why = f"NVML: {type(e).__name__}: {e}"

    def _fields(self, scopes):
        nv = self.nv
        ids = [(f, s) for s in scopes for f in (nv.NVML_FI_DEV_NVLINK_THROUGHPUT_DATA_TX,
                                                nv.NVML_FI_DEV_NVLINK_THROUGHPUT_DATA_RX)]
        vals = nv.nvmlDeviceGetFieldValues(self.handle, ids)
        good = [v for v in vals if v.nvmlReturn == nv.NVML_SUCCESS]
        if not good:
            self.why = f"field query returned {sorted({int(v.nvmlReturn) for v in vals})}"
            return None
        tx = sum(int(v.value.ullVal) for v in good if v.fieldId == nv.NVML_FI_DEV_NVLINK_THROUGHPUT_DATA_TX)
        rx = sum(int(v.value.ullVal) for v in good if v.fieldId == nv.NVML_FI_DEV_NVLINK_THROUGHPUT_DATA_RX)
        return tx * 1024, rx * 1024

    def read(self):
        if self.handle is None:
            return None
        try:
            if not self.per_link:
                got = self._fields([0xFFFFFFFF])   # scope: all links of the device
                if got is not None:
                    return got
                self.per_link = True
            return self._fields(range(18))
        except Exception as e:
            self.why = f"{type(e).__name__}: {e}"
            return None


def emit(record: dict) -> None:
    world, rank = world_rank()
    if rank == 0:
        print(json.dumps(record), flush=True)
