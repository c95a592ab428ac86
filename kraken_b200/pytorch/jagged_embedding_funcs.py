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
    the same kernel sequence) and one fused push.  GPU engine only.  The first argument is the
    table's (empty) Parameter: it is what makes autograd call ``backward``."""

    @staticmethod
    def forward(ctx, sparse_table, values, offsets, weights, mean, patch_value):
        eng = native.engine()
        tid = sparse_table.table_id()
        out, ticket = eng.pull_sparse_pooled(tid, values, offsets, weights=weights, mean=mean, patch_value=patch_value)
        ctx.table_id, ctx.ticket, ctx.values = tid, ticket, values
        return out

    @staticmethod
    def backward(ctx, grads):
        native.engine().push_sparse_pooled(ctx.table_id, ctx.ticket, grads.contiguous(), ctx.values)
        return None, None, None, None, None, None


class FusedCombineJaggedLookupFunction(torch.autograd.Function):
    """Bags of several tables pooled through the combined exchange: tables of equal row width (and equal
    patch value) share one dedup, one dispatch, one pooled gather and one push
    (kraken/pytorch/combine_jagged_embedding.py:11-76 over kraken/worker/emitter.cc:185-278).
    ``inputs`` is a list of (values, offsets, weights-or-None) per table."""

    @staticmethod
    def forward(ctx, combine_sparse_table, inputs, means, patch_values):
        eng = native.engine()
        outs, handles = eng.combine_pull_sparse_pooled(combine_sparse_table.table_ids(), inputs, means, patch_values)
        ctx.handles = handles
        return tuple(outs)

    @staticmethod
    def backward(ctx, *grads):
        native.engine().combine_push_sparse_pooled(ctx.handles, list(grads))
        return None, None, None, None
