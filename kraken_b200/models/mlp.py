"""Multi-layer perceptron head (Linear + ReLU, no activation after the last layer)."""
from __future__ import annotations

from typing import Sequence

import torch


class MLP(torch.nn.Module):
    def __init__(self, in_features: int, sizes: Sequence[int]):
        super().__init__()
        layers = []
        prev = in_features
        for n in sizes:
            layers.append(torch.nn.Linear(prev, n))
            prev = n
        self.layers = torch.nn.ModuleList(layers)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        last = len(self.layers) - 1
        for i, layer in enumerate(self.layers):
            x = layer(x)
            if i != last:
                x = torch.relu(x)
        return x
