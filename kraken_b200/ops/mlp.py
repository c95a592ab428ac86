"""MLP head on the tcgen05 Linear kernels (csrc/cuda/mlp_gemm.cu).

``fused_mlp(x, weights, biases)`` runs Linear+ReLU layers on bf16 activations
with fp32 parameters and fp32 accumulation; the last layer has no activation
and, when it has a single output, runs as a row-dot kernel that keeps the
logit in fp32.  The backward pass is hand-scheduled: per layer one split-K
weight-gradient GEMM that red-adds straight into the parameter's gradient
buffer, one column-sum for the bias and one input-gradient GEMM with the ReLU
mask of the previous layer fused into its epilogue.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from .._native import C
from . import counters

_status = {}
_side_streams = {}
_deferred_join = False
_pending_join = set()


_grad_ready = None


def set_grad_ready_callback(fn) -> None:
    """``fn(parameter, stream)`` is called by the backward pass once every kernel that writes a parameter's
    gradient this step has been enqueued on ``stream`` (the engine uses it to launch the fused dense step of a
    bucket while the backward pass is still running)."""
    global _grad_ready
    _grad_ready = fn


def _notify(params, stream) -> None:
    if _grad_ready is not None:
        for p in params:
            _grad_ready(p, stream)


def set_deferred_join(on: bool) -> None:
    """With deferred join the backward pass leaves its side stream (weight and bias gradients)
    un-joined, and whoever consumes those gradients next - the engine's fused dense step - runs on
    that stream and joins it afterwards.  The sparse backward and push that follow the MLP in a
    recommender's backward pass then run beside the last weight gradients and the dense step
    instead of behind them.  Only safe when nothing reads ``param.grad`` of the MLP on the main
    stream before the dense step, which is why the engine option that turns it on is off by default."""
    global _deferred_join
    _deferred_join = bool(on)
    if not on:
        _pending_join.clear()


def take_pending_side_stream(device: torch.device) -> Optional[torch.cuda.Stream]:
    """The side stream with un-joined gradient work on ``device`` (and marks it as taken), or None."""
    key = (device.type, device.index)
    if key in _pending_join:
        _pending_join.discard(key)
        return _side_streams.get(key)
    return None


def _side_stream(device: torch.device) -> torch.cuda.Stream:
    """Second stream on which weight and bias gradients run beside the input-gradient chain."""
    key = (device.type, device.index)
    if key not in _side_streams:
        _side_streams[key] = torch.cuda.Stream(device=device)
    return _side_streams[key]



class PreparedWeights:
    """bf16 copies of the hidden layers' weights (both layouts), cast on the side stream."""

    def __init__(self, w16s, wt16s, event):
        self.w16s, self.wt16s, self.event = w16s, wt16s, event


def prepare_weights(weights: Sequence[torch.Tensor]) -> PreparedWeights:
    """Starts the fp32 -> bf16 casts of the hidden layers' weights on the side stream and returns
    at once.  A model calls this before work that does not depend on the weights (the sparse
    pull of a recommender), hands the result to ``fused_mlp(prepared=...)``, and the casts run
    beside that work instead of in front of the first GEMM."""
    dev = weights[0].device
    main = torch.cuda.current_stream(dev)
    side = _side_stream(dev)
    side.wait_stream(main)
    w16s, wt16s = [], []
    with torch.cuda.stream(side):
        for w in weights[:-1]:
            counters.add()
            w16, wt16 = C.cast_w_wt(w.detach().contiguous())
            w16.record_stream(main)
            wt16.record_stream(main)
            w16s.append(w16)
            wt16s.append(wt16)
        event = torch.cuda.Event()
        event.record(side)
    return PreparedWeights(w16s, wt16s, event)


def gemm_status(device: torch.device) -> torch.Tensor:
    """Device word in which the GEMM kernels record a pipeline wait that gave up."""
    key = (device.type, device.index)
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status[key]


def check_gemm_status(device: torch.device) -> None:
    st = gemm_status(device)
    code = int(st.item())
    if code != 0:
        st.zero_()
        raise C.KrakenError(f"tcgen05 GEMM: {C.error_message(code)} (code {code})")


def supported(in_features: int, sizes: Sequence[int]) -> bool:
    """Whether the hidden layers meet the TMA pitch rule (widths in multiples of 8 elements).
    The last layer may have any width: 1 runs as a row-dot kernel, a multiple of 8 on the
    tensor cores, anything else (a 10-class head, say) as a small fp32 matmul."""
    dims = [in_features] + list(sizes)
    return len(sizes) >= 1 and all(d % 8 == 0 for d in dims[:-1])


def _grad_target(p: torch.Tensor) -> torch.Tensor:
    """The buffer a parameter's gradient is accumulated into (created zeroed if absent)."""
    if p.grad is None:
        p.grad = torch.zeros_like(p)
    return p.grad


class _FusedMLP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, addend, n_layers, input_grad_cols, prepared, *params):
        ws, bs = params[:n_layers], params[n_layers:]
        dev = x.device
        if prepared is not None:
            torch.cuda.current_stream(dev).wait_event(prepared.event)
        st = gemm_status(dev)
        h = x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)
        acts = [h]
        M = h.shape[0]
        wts = []
        masks = [None]  # masks[i] belongs to acts[i]; the MLP input has none
        for i in range(n_layers - 1):
            if prepared is not None:
                w16, wt16 = prepared.w16s[i], prepared.wt16s[i]
            else:
                counters.add()
                w16, wt16 = C.cast_w_wt(ws[i].detach().contiguous())  # both layouts in one pass; wt16 is for backward
            wts.append(wt16)
            y = torch.empty((M, w16.shape[0]), dtype=torch.bfloat16, device=dev)
            # one bit per output (> 0): the next layer's input gradient masks with it instead of re-reading y
            mask = torch.empty(((w16.shape[0] + 15) // 16, (M + 63) // 64 * 64), dtype=torch.int16, device=dev)
            counters.add()
            C.linear_forward(h, w16, bs[i].detach(), True, y, st, mask)
            acts.append(y)
            masks.append(mask)
            h = y
        wl, bl = ws[-1].detach(), bs[-1].detach()
        if wl.shape[0] == 1:
            out = torch.empty(M, dtype=torch.float32, device=dev)
            counters.add()
            C.rowdot_forward(h, wl.reshape(-1).contiguous(), bl, out,
                             addend.detach().float().contiguous() if addend is not None else None)
            out = out.view(M, 1)
            addend = None
        elif wl.shape[0] % 8 == 0:
            y = torch.empty((M, wl.shape[0]), dtype=torch.bfloat16, device=dev)
            counters.add()
            C.linear_forward(h, wl.to(torch.bfloat16), bl, False, y, st)
            out = y.float()
        else:
            out = torch.addmm(bl, h.float(), wl.t())  # narrow odd-width head: library fp32 matmul
        if addend is not None:
            out = out + addend.reshape(M, 1).to(out.dtype)
        ctx.acts, ctx.ws, ctx.bs, ctx.n_layers, ctx.wts, ctx.masks = acts, ws, bs, n_layers, wts, masks
        ctx.x_needs_grad = x.requires_grad
        ctx.input_grad_cols = input_grad_cols
        ctx.x_dtype = x.dtype
        return out

    @staticmethod
    def backward(ctx, gout):
        from ..utils.profiler import engine_region
        with engine_region("mlp_bwd"):
            return _FusedMLP._backward(ctx, gout)

    @staticmethod
    def _backward(ctx, gout):
        acts, ws, bs, L = ctx.acts, ctx.ws, ctx.bs, ctx.n_layers
        dev = gout.device
        st = gemm_status(dev)
        M = acts[0].shape[0]
        wl = ws[-1]
        h_last = acts[-1]
        need_dx_last = L > 1 or ctx.x_needs_grad
        if wl.shape[0] == 1:
            dy = gout.reshape(-1).float().contiguous()
            dh = torch.empty_like(h_last) if need_dx_last else None
            counters.add()
            C.rowdot_backward(h_last, wl.detach().reshape(-1).contiguous(), dy, L > 1, dh,
                              _grad_target(wl).view(-1), _grad_target(bs[-1]))
        elif wl.shape[0] % 8 != 0:
            g32 = gout.float()
            h32 = h_last.float()
            _grad_target(wl).addmm_(g32.t(), h32)
            _grad_target(bs[-1]).add_(g32.sum(0))
            dh = None
            if need_dx_last:
                d = g32 @ wl.detach()
                if L > 1:
                    d = d * (h32 > 0)
                dh = d.to(torch.bfloat16)
        else:
            dy16 = gout.to(torch.bfloat16).contiguous()
            counters.add()
            C.linear_wgrad(dy16, h_last, _grad_target(wl), st)
            counters.add()
            C.colsum_bf16(dy16, _grad_target(bs[-1]))
            dh = None
            if need_dx_last:
                dh = torch.empty_like(h_last)
                counters.add()
                C.linear_dgrad(dy16, wl.detach().t().contiguous().to(torch.bfloat16), None, dh, st,
                               ctx.masks[-1] if L > 1 else None)
        _notify((wl, bs[-1]), torch.cuda.current_stream(dev))
        # The chain dh_L -> dh_{L-1} -> ... is serial; each layer's weight and bias gradients only
        # need that layer's dh, so they run on a second stream beside the chain and are joined at
        # the end (in a CUDA-graph capture this becomes a parallel branch).
        main = torch.cuda.current_stream(dev)
        side = _side_stream(dev)
        for i in range(L - 2, -1, -1):
            # dh is d(loss)/d(acts[i + 1]) with layer i's ReLU mask already applied
            side.wait_stream(main)
            with torch.cuda.stream(side):
                counters.add(2)
                C.linear_wgrad(dh, acts[i], _grad_target(ws[i]), st)
                C.colsum_bf16(dh, _grad_target(bs[i]))
                dh.record_stream(side)
            _notify((ws[i], bs[i]), side)
            if i > 0 or ctx.x_needs_grad:
                dprev = torch.empty_like(acts[i])
                wt16 = ctx.wts[i]
                counters.add()
                cols = ctx.input_grad_cols if (i == 0 and ctx.input_grad_cols) else dprev.shape[1]
                if cols < dprev.shape[1]:
                    # only the leading columns of the input need a gradient (the rest are constants)
                    dprev[:, cols:].zero_()
                    C.linear_dgrad(dh, wt16[:cols], None, dprev[:, :cols], st)
                else:
                    C.linear_dgrad(dh, wt16, None, dprev, st, ctx.masks[i])
                dh = dprev
            else:
                dh = None
        if _deferred_join:
            _pending_join.add((dev.type, dev.index))
        else:
            main.wait_stream(side)
        dx = None
        if ctx.x_needs_grad and dh is not None:
            dx = dh if ctx.x_dtype == torch.bfloat16 else dh.to(ctx.x_dtype)
        # parameter gradients were accumulated in place
        return (dx, gout.reshape(-1) if ctx.needs_input_grad[1] else None, None, None, None) + (None,) * (2 * L)


def fused_mlp(x: torch.Tensor, weights: List[torch.Tensor], biases: List[torch.Tensor],
              input_grad_cols: int = 0, addend: Optional[torch.Tensor] = None,
              prepared: Optional[PreparedWeights] = None) -> torch.Tensor:
    """x [M, K] (bf16 or fp32, CUDA) -> [M, out_features] fp32.  Parameter gradients are
    accumulated into ``param.grad`` in place by the backward kernels.  ``input_grad_cols``
    (a multiple of 8, 0 = all) limits the input gradient to the leading columns of x.
    ``addend`` [M] (single-output heads) is added to the output inside the head kernel.
    ``prepared`` is the result of an earlier ``prepare_weights`` call on the same weights."""
    from ..utils.profiler import engine_region
    with engine_region("mlp_fwd"):
        if addend is not None and weights[-1].shape[0] != 1:
            raise ValueError("addend needs a single-output head")
        return _FusedMLP.apply(x, addend, len(weights), int(input_grad_cols), prepared, *weights, *biases)
