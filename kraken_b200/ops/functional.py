"""Autograd front ends of the model kernels (csrc/cuda/model_kernels.cu).

On CUDA tensors the hand-written kernels run and there is no fallback; on CPU
tensors the same math is expressed with torch ops, which is also what the
tests use as the fp32 oracle.
"""
from __future__ import annotations

import torch

from .._native import C
from . import counters


class _FMInteraction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, emb):
        emb = emb.contiguous()
        ctx.save_for_backward(emb)
        counters.add()
        return C.fm_forward(emb)

    @staticmethod
    def backward(ctx, gout):
        (emb,) = ctx.saved_tensors
        counters.add()
        return C.fm_backward(emb, gout.contiguous())


def fm_interaction(emb: torch.Tensor) -> torch.Tensor:
    """FM second-order term of emb [B, F, D]: 0.5 * sum_d((sum_f e)^2 - sum_f e^2) -> [B]
    (the expression of examples/DeepFM/model/DeepFM.py:96-107, summed over d)."""
    if emb.is_cuda:
        return _FMInteraction.apply(emb.float())
    s = emb.sum(1)
    return 0.5 * (s * s - (emb * emb).sum(1)).sum(1)


class _BCEWithLogits(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, labels):
        counters.add()
        loss, grad = C.bce_with_logits(logits.contiguous().view(-1), labels.contiguous().view(-1).float(), True)
        ctx.save_for_backward(grad)
        ctx.shape = logits.shape
        return loss

    @staticmethod
    def backward(ctx, gout):
        (grad,) = ctx.saved_tensors
        return (grad * gout).view(ctx.shape), None


def bce_with_logits(logits: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
    """Mean binary cross entropy on logits (forward and gradient in one kernel pass)."""
    if logits.is_cuda:
        return _BCEWithLogits.apply(logits.float(), labels)
    return torch.nn.functional.binary_cross_entropy_with_logits(logits, labels.float())
