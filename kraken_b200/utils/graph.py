"""CUDA-graph replay of a whole training step.

At small per-GPU batches a step is a few dozen short kernels and the time goes
to launching them, not to running them.  Every kernel of this framework takes
its per-step scalars (learning rate, exchange epochs, step counters) from
device memory and never synchronises the host, so one step - sparse pull,
model forward and backward, sparse push, fused dense update - can be captured
once and replayed: ``GraphedStep`` does that.

    step = GraphedStep(lambda dense, ids, labels: train_step(dense, ids, labels), example_batch)
    loss = step(dense, ids, labels)      # copies the inputs into static buffers and replays

The captured function must run the same kernel sequence every step.  What a
step does on the host is not part of a graph, so after every replay
``GraphedStep`` runs it itself: ``optimizer.host_step()`` when an optimizer was
given (learning-rate schedule into the engine's device-side value), else the
engine's ``end_step()`` - table growth and the kernels' error words.  When a
table had to be reallocated the captured graphs hold stale pointers and are
captured again before the next replay.  DCT's periodic threshold refresh is
not capturable.  Every rank of a multi-GPU job captures its own graph and
replays in lockstep; the cross-GPU waits inside the kernels stay bounded.
"""
from __future__ import annotations

from typing import Callable, Sequence

import torch


class GraphedStep:
    def __init__(self, fn: Callable, example_inputs: Sequence[torch.Tensor], warmup: int = 3,
                 device: torch.device | None = None, slots: int = 1, optimizer=None) -> None:
        """slots > 1 captures the step once per set of static input buffers (the graphs share one
        memory pool, they never run at the same time).  An input pipeline can then fill the buffers
        of slot k + 1 while slot k is being replayed (``static_inputs`` / ``replay`` /
        ``launch_slot``), so no device-to-device copy of the inputs is needed."""
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.fn = fn
        self.optimizer = optimizer
        self.recaptures = 0
        self.slots = max(1, int(slots))
        self.static_ins = [[torch.empty(t.shape, dtype=t.dtype, device=self.device) for t in example_inputs]
                           for _ in range(self.slots)]
        for bufs in self.static_ins:
            for s, t in zip(bufs, example_inputs):
                s.copy_(t)
        self.static_in = self.static_ins[0]
        # eager warm-up on a side stream: creates channels / buckets and fills the allocator pool
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            for _ in range(max(1, warmup)):
                fn(*self.static_in)
        torch.cuda.current_stream(self.device).wait_stream(side)
        self._capture()

    def _capture(self) -> None:
        torch.cuda.synchronize(self.device)
        self.graphs, self.static_outs = [], []
        for k in range(self.slots):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, pool=self.graphs[0].pool() if self.graphs else None):
                out = self.fn(*self.static_ins[k])
            self.graphs.append(g)
            self.static_outs.append(out)
            torch.cuda.synchronize(self.device)
        self.graph, self.static_out = self.graphs[0], self.static_outs[0]

    def _after_replay(self) -> None:
        """Host-side work of a step (see the module text); rebuilds the graphs after a table grew."""
        if self.optimizer is not None:
            grew = self.optimizer.host_step()
        else:
            from ..pytorch import native
            grew = bool(native.engine().end_step()) if native.is_initialized() and hasattr(native.engine(), "end_step") else False
        if grew:
            self.recaptures += 1
            self._capture()

    def __call__(self, *inputs: torch.Tensor):
        for s, t in zip(self.static_in, inputs):
            s.copy_(t, non_blocking=True)
        self.graph.replay()
        out = self.static_out
        self._after_replay()
        return out

    def static_inputs(self, slot: int):
        """The input buffers that the graph of ``slot`` reads."""
        return tuple(self.static_ins[slot])

    def replay(self, slot: int = 0):
        """Replays the graph of ``slot`` on whatever its input buffers hold now."""
        self.graphs[slot].replay()
        out = self.static_outs[slot]
        self._after_replay()
        return out

    def launch_slot(self, slot: int) -> "PendingScalar":
        """``replay(slot)`` plus the start of the (scalar) result's copy to pinned host memory."""
        return self._pending(self.replay(slot))

    def _pending(self, out: torch.Tensor) -> "PendingScalar":
        if not hasattr(self, "_slots"):
            self._slots = [PendingScalar(out) for _ in range(4)]
            self._next = 0
        slot = self._slots[self._next]
        self._next = (self._next + 1) % len(self._slots)
        slot.capture(out)
        return slot

    def launch(self, *inputs: torch.Tensor) -> "PendingScalar":
        """Replays the step and starts copying its (scalar) result to pinned host memory without
        waiting for it: the caller can enqueue the next step first and read this step's value
        afterwards, so the device never idles on the host's round trip.

            pending = None
            for batch in loader:
                h = step.launch(*batch)
                if pending is not None:
                    log(pending.item())
                pending = h
        """
        return self._pending(self(*inputs))


class PendingScalar:
    """A device scalar on its way to pinned host memory; ``item()`` waits for that copy only."""

    def __init__(self, like: torch.Tensor) -> None:
        self.host = torch.empty(like.shape, dtype=like.dtype).pin_memory()
        self.event = torch.cuda.Event()

    def capture(self, value: torch.Tensor) -> None:
        self.host.copy_(value, non_blocking=True)
        self.event.record()

    def item(self) -> float:
        self.event.synchronize()
        return self.host.item()
