"""Autograd wrappers of the jagged (bag) pooling kernels, CPU and CUDA
(kraken/pytorch/jagged_embedding_funcs.py:7-34).  Unlike the reference's sum
backward, every row of a bag receives the bag's gradient."""
import torch

from . import native


class JaggedEmbeddingSumFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, values, offsets, patch_value):
        ctx.save_for_backward(offsets)
        return native.jagged_sum_forward(values, offsets, patch_value)

    @staticmethod
    def backward(ctx, grads):
        (offsets,) = ctx.saved_tensors
        return native.jagged_sum_backward(offsets, grads.contiguous()), None, None


class JaggedEmbeddingMeanFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, values, offsets, patch_value):
        ctx.save_for_backward(offsets)
        return native.jagged_mean_forward(values, offsets, patch_value)

    @staticmethod
    def backward(ctx, grads):
        (offsets,) = ctx.saved_tensors
        return native.jagged_mean_backward(offsets, grads.contiguous()), None, None


class FusedJaggedLookupFunction(torch.autograd.Function):
    """EmbeddingBag as one fused pull (dedup, exchange, gather and pooling in
    the same kernel sequence) and one fused push.  GPU engine only."""

    @staticmethod
    def forward(ctx, sparse_table_id, values, offsets, weights, mean, patch_value):
        eng = native.engine()
        out, ticket = eng.pull_sparse_pooled(sparse_table_id, values, offsets, weights=weights, mean=mean,
                                             patch_value=patch_value)
        ctx.table_id, ctx.ticket, ctx.values = sparse_table_id, ticket, values
        return out

    @staticmethod
    def backward(ctx, grads):
        native.engine().push_sparse_pooled(ctx.table_id, ctx.ticket, grads.contiguous(), ctx.values)
        return None, None, None, None, None, None
