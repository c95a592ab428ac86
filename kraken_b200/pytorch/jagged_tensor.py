"""JaggedTensor: a batch of variable-length bags stored as (values, offsets[, weights]).

Bag b holds ``values[offsets[b]:offsets[b + 1]]``.  Same constructor, accessors
and ``from_list_tensors`` as kraken/pytorch/jagged_tensor.py:7-89; the optional
weights are tested with ``is not None`` (the reference's truth test of a tensor
fails for more than one element).
"""
from typing import List, Optional

import torch


class JaggedTensor(object):
    def __init__(self, values: torch.Tensor, offsets: torch.Tensor, weights: Optional[torch.Tensor] = None,
                 validate: bool = True):
        if validate:
            self._check_params(values, offsets, weights)
        self._values = values
        self._offsets = offsets
        self._weights = weights

    def values(self) -> torch.Tensor:
        return self._values

    def offsets(self) -> torch.Tensor:
        return self._offsets

    def weights(self) -> Optional[torch.Tensor]:
        return self._weights

    def num_bags(self) -> int:
        return int(self._offsets.numel()) - 1

    @staticmethod
    def _check_params(values, offsets, weights=None):
        off = offsets.tolist()
        if len(off) < 1 or off[0] != 0 or off[-1] != values.shape[0]:
            raise ValueError(f"JaggedTensor offsets are invalid: {off}, values shape: {tuple(values.shape)}")
        for a, b in zip(off, off[1:]):
            if b < a:
                raise ValueError(f"JaggedTensor offsets must not decrease: {off}")
        if weights is not None and weights.shape != values.shape:
            raise ValueError(f"JaggedTensor needs values and weights of the same shape, got "
                             f"{tuple(weights.shape)} and {tuple(values.shape)}")

    @staticmethod
    def from_list_tensors(list_values: List[torch.Tensor], list_weights: Optional[List[torch.Tensor]] = None):
        if len(list_values) == 0:
            raise ValueError("from_list_tensors needs at least one tensor")
        tail = list_values[0].shape[1:]
        offs = [0]
        for v in list_values:
            if v.shape[1:] != tail:
                raise ValueError("JaggedTensor needs values with the same shape except for the first dimension")
            offs.append(offs[-1] + v.shape[0])
        weights = None
        if list_weights is not None:
            if len(list_weights) != len(list_values):
                raise ValueError("one weight tensor per value tensor is required")
            for v, w in zip(list_values, list_weights):
                if v.shape != w.shape:
                    raise ValueError("JaggedTensor needs values and weights of the same shape")
            weights = torch.cat(list_weights, 0)
        return JaggedTensor(values=torch.cat(list_values, 0), offsets=torch.as_tensor(offs, dtype=torch.int64),
                            weights=weights)
