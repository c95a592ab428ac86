"""One-batch-ahead host-to-device input pipeline.

The reference's workers read their batches with a torch ``DataLoader`` on the
host and hand them to the model synchronously (examples/deepfm/main.py of the
reference); on a B200 the 17 MB of ids of a 65,536-sample DeepFM batch take
longer to cross PCIe than a fifth of the step, so the copy of batch ``i+1``
runs on its own stream while batch ``i`` trains.

    for dense, ids, labels in DevicePrefetcher(loader, device):
        loss = step(dense, ids, labels)

``loader`` yields tuples of pinned host tensors of fixed shapes.  Two sets of
device buffers are used in turn; a buffer is refilled only after the step that
read it has been enqueued behind an event, so no batch is overwritten early.
"""
from __future__ import annotations

from typing import Iterable, Iterator, List, Optional, Sequence, Tuple

import torch


class DevicePrefetcher:
    def __init__(self, loader: Iterable[Sequence[torch.Tensor]], device: torch.device, depth: int = 2,
                 chunk_bytes: int = 1 << 18, buffers: Optional[Sequence[Sequence[torch.Tensor]]] = None) -> None:
        """buffers: device buffer sets to fill in turn instead of allocating (for instance the static
        inputs of a multi-slot ``GraphedStep``; ``last_slot`` then tells which set a batch landed in).
        chunk_bytes: large tensors cross PCIe as a series of copies of at most this size.  One long
        DMA transfer of 17 MB running beside the step's kernels was measured to slow a 1.03 ms step by
        0.24 ms, 1 MB pieces by 0.14 ms, 256 KB pieces by 0.06 ms; at 64 KB the host cannot issue
        the copies fast enough."""
        self.chunk_bytes = max(1 << 16, int(chunk_bytes))
        self.it: Iterator[Sequence[torch.Tensor]] = iter(loader)
        self.device = device
        self.depth = max(2, depth) if buffers is None else len(buffers)
        if self.depth < 2:
            raise ValueError("a prefetcher needs at least two buffer sets")
        self.copy_stream = torch.cuda.Stream(device=device)
        self.bufs: List[Optional[Tuple[torch.Tensor, ...]]] = [None] * self.depth
        if buffers is not None:
            self.bufs = [tuple(b) for b in buffers]
        self.last_slot = -1
        self.ready = [torch.cuda.Event() for _ in range(self.depth)]     # copy into slot finished
        self.released = [torch.cuda.Event() for _ in range(self.depth)]  # consumer of slot enqueued its work
        self.used = [False] * self.depth
        self.head = 0  # next slot to fill
        self.tail = 0  # next slot to hand out
        self.pending = 0
        self.bytes_copied = 0
        self._fill()

    def _fill(self) -> bool:
        try:
            host = next(self.it)
        except StopIteration:
            return False
        slot = self.head
        if self.bufs[slot] is None:
            self.bufs[slot] = tuple(torch.empty(t.shape, dtype=t.dtype, device=self.device) for t in host)
        with torch.cuda.stream(self.copy_stream):
            if self.used[slot]:
                self.copy_stream.wait_event(self.released[slot])
            for d, h in zip(self.bufs[slot], host):
                nbytes = h.numel() * h.element_size()
                self.bytes_copied += nbytes
                if nbytes <= self.chunk_bytes or not (h.is_contiguous() and d.is_contiguous()):
                    d.copy_(h, non_blocking=True)
                    continue
                dv, hv = d.view(-1), h.view(-1)
                per = max(1, self.chunk_bytes // h.element_size())
                for a in range(0, hv.numel(), per):
                    dv[a:a + per].copy_(hv[a:a + per], non_blocking=True)
            self.ready[slot].record(self.copy_stream)
        self.head = (slot + 1) % self.depth
        self.pending += 1
        return True

    def __iter__(self) -> "DevicePrefetcher":
        return self

    def __next__(self) -> Tuple[torch.Tensor, ...]:
        if self.pending == 0:
            raise StopIteration
        main = torch.cuda.current_stream(self.device)
        # the slot handed out before this one is free again once the work enqueued so far has run
        prev = (self.tail - 1) % self.depth
        if self.used[prev]:
            self.released[prev].record(main)
        slot = self.tail
        main.wait_event(self.ready[slot])
        self.used[slot] = True
        self.last_slot = slot
        self.tail = (slot + 1) % self.depth
        self.pending -= 1
        while self.pending < self.depth - 1 and self._fill():
            pass
        return self.bufs[slot]  # type: ignore[return-value]
