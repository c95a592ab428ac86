"""Multi-layer perceptron head (Linear + ReLU, no activation after the last layer).

On CUDA, when every layer width is a multiple of 8, the layers run on the
hand-written tcgen05 kernels in bf16 with fp32 accumulation
(``kraken_b200.ops.mlp``); otherwise, and on CPU, plain torch ops are used.
"""
from __future__ import annotations

from typing import Sequence

import torch

from ..ops import mlp as fused


class MLP(torch.nn.Module):
    def __init__(self, in_features: int, sizes: Sequence[int], use_tensor_cores: bool = True):
        super().__init__()
        layers = []
        prev = in_features
        for n in sizes:
            layers.append(torch.nn.Linear(prev, n))
            prev = n
        self.layers = torch.nn.ModuleList(layers)
        self.in_features = in_features
        self.sizes = list(sizes)
        self.use_tensor_cores = use_tensor_cores and fused.supported(in_features, sizes)

    def prepare(self):
        """Starts casting the weights for the tensor-core path on a side stream (CUDA only); pass
        the result as ``prepared`` to ``forward``.  Returns None where there is nothing to do."""
        w = self.layers[0].weight
        if w.is_cuda and self.use_tensor_cores and len(self.layers) > 1:
            return fused.prepare_weights([l.weight for l in self.layers])
        return None

    def forward(self, x: torch.Tensor, input_grad_cols: int = 0, addend=None, prepared=None) -> torch.Tensor:
        """addend [M]: added to a single-output head (fused into the head kernel on CUDA)."""
        if x.is_cuda and self.use_tensor_cores:
            return fused.fused_mlp(x, [l.weight for l in self.layers], [l.bias for l in self.layers],
                                   input_grad_cols if input_grad_cols % 8 == 0 else 0, addend, prepared)
        if addend is not None:
            return self.forward(x) + addend.reshape(-1, 1)
        x = x.float()
        last = len(self.layers) - 1
        for i, layer in enumerate(self.layers):
            x = layer(x)
            if i != last:
                x = torch.relu(x)
        return x
