"""CUDA-graph replay of a whole training step.

At small per-GPU batches a step is a few dozen short kernels and the time goes
to launching them, not to running them.  Every kernel of this framework takes
its per-step scalars (learning rate, exchange epochs, step counters) from
device memory and never synchronises the host, so one step - sparse pull,
model forward and backward, sparse push, fused dense update - can be captured
once and replayed: ``GraphedStep`` does that.

    step = GraphedStep(lambda dense, ids, labels: train_step(dense, ids, labels), example_batch)
    loss = step(dense, ids, labels)      # copies the inputs into static buffers and replays

The captured function must run the same kernel sequence every step: tables
must be sized so that they do not grow inside the step (growth is checked
between replays by ``engine.end_step()``), the learning rate must change only
through the engine's device-side value, and DCT's periodic threshold refresh
is not capturable.  Every rank of a multi-GPU job captures its own graph and
replays in lockstep; the cross-GPU waits inside the kernels stay bounded.
"""
from __future__ import annotations

from typing import Callable, Sequence

import torch


class GraphedStep:
    def __init__(self, fn: Callable, example_inputs: Sequence[torch.Tensor], warmup: int = 3,
                 device: torch.device | None = None) -> None:
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.static_in = [torch.empty(t.shape, dtype=t.dtype, device=self.device) for t in example_inputs]
        for s, t in zip(self.static_in, example_inputs):
            s.copy_(t)
        # eager warm-up on a side stream: creates channels / buckets and fills the allocator pool
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            for _ in range(max(1, warmup)):
                fn(*self.static_in)
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            out = fn(*self.static_in)
        self.static_out = out
        torch.cuda.synchronize(self.device)

    def __call__(self, *inputs: torch.Tensor):
        for s, t in zip(self.static_in, inputs):
            s.copy_(t, non_blocking=True)
        self.graph.replay()
        return self.static_out
