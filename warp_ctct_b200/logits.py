"""CTC-Transducer loss on raw joint logits: ``ctct_loss(log_softmax(logits, -1), ...)`` with the
log-softmax fused into the loss kernels (no counterpart in the reference, whose callers run
``log_softmax`` themselves before ``warp_ctct.ctct_loss``, warp_ctct/__init__.py:97-100).

Forward: one streaming read of the valid rows gives every row's log-sum-exp and the three
log-probs the lattice needs.  Backward: one pass writes
``d loss / d logits = G - softmax(logits) * sum(G)`` (G: the <= 3 occupancy-gradient entries of a
row), reading valid rows once more and writing every row once.  Nothing of the size of the joint
tensor is allocated besides the gradient itself.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib

T = torch.Tensor


def _forward(ctx, logits: T, labels: T, lx: T, ly: T, requires_grad: bool, red: int, average_frames: bool, norm: float):
    from . import PREZERO, PREZERO_MIN_BYTES, _sizes
    N, Tm, U1, V = logits.shape
    dev = logits.device
    lib = _lib.lib()
    g3_bytes, ws_bytes = _sizes(N, Tm, U1, requires_grad)
    with _lib.on_device(dev):
        out = torch.empty((N + 1,), dtype=torch.float32, device=dev)
        buf = torch.empty((g3_bytes + ws_bytes,), dtype=torch.uint8, device=dev)  # [compact gradient | workspace]
        # The gradient buffer is allocated now so that the lattice launch can zero its padding rows
        # (nothing the loss computes is needed for that) while the recursion, which is latency-bound, runs.
        grad = None
        if (requires_grad and PREZERO and logits.numel() * logits.element_size() >= PREZERO_MIN_BYTES
                and (V * logits.element_size()) % 16 == 0):
            grad = torch.empty_like(logits)
        base = buf.data_ptr()
        rc = lib.ctct_b200_logits_forward(
            logits.data_ptr(), _lib.dtype_code(logits.dtype), labels.data_ptr(), lx.data_ptr(), ly.data_ptr(),
            N, Tm, U1, V, int(requires_grad), red, int(average_frames), norm, out.data_ptr() + 4, out.data_ptr(),
            base if requires_grad else None, _lib.ptr(grad), base + g3_bytes, ws_bytes, _lib.raw_stream(dev))
    _lib.check(rc, "ctct_b200_logits_forward")
    if requires_grad:
        ctx.save_for_backward(buf, logits, labels, lx, ly)
        ctx.meta = (N, Tm, U1, V, red, bool(average_frames), float(norm))
        ctx.cleared = grad
    return out


def _backward(ctx, grad: T) -> T:
    buf, logits, labels, lx, ly = ctx.saved_tensors
    N, Tm, U1, V, red, avg, norm = ctx.meta
    dev = logits.device
    go = grad.to(torch.float32).contiguous()
    out, ctx.cleared = ctx.cleared, None   # a second backward through a retained graph gets a fresh buffer
    cleared = out is not None
    with _lib.on_device(dev):
        if out is None:
            out = torch.empty_like(logits)
        rc = _lib.lib().ctct_b200_logits_backward(
            buf.data_ptr(), go.data_ptr(), int(red != 0), red, int(avg), norm, logits.data_ptr(), labels.data_ptr(),
            lx.data_ptr(), ly.data_ptr(), N, Tm, U1, V, _lib.dtype_code(logits.dtype), out.data_ptr(), int(cleared),
            _lib.raw_stream(dev))
    _lib.check(rc, "ctct_b200_logits_backward")
    return out


class FusedLogitsCTCTLoss(torch.autograd.Function):
    """Per-utterance costs from raw logits (N,T,U+1,V); gradient w.r.t. the logits."""

    @staticmethod
    def forward(ctx, logits: T, labels: T, lx: T, ly: T, requires_grad: bool):
        return _forward(ctx, logits, labels, lx, ly, requires_grad, 0, False, 1.0)[1:]

    @staticmethod
    def backward(ctx, grad_outputs: T):
        return _backward(ctx, grad_outputs), None, None, None, None


class FusedLogitsCTCTLossReduced(torch.autograd.Function):
    """The same with the 'sum' / 'mean' reduction (and average_frames) folded into the kernels."""

    @staticmethod
    def forward(ctx, logits: T, labels: T, lx: T, ly: T, requires_grad: bool, mean: bool, average_frames: bool,
                norm: float):
        return _forward(ctx, logits, labels, lx, ly, requires_grad, 2 if mean else 1, bool(average_frames), float(norm))[0]

    @staticmethod
    def backward(ctx, grad_loss: T):
        return _backward(ctx, grad_loss), None, None, None, None, None, None, None


def ctct_loss_from_logits(logits: T, labels: T, frames_lengths: T, labels_lengths: T,
                          reduction: Optional[str] = "mean", average_frames: bool = False,
                          global_batch: Optional[int] = None) -> T:
    """``ctct_loss(logits.log_softmax(-1), labels, frames_lengths, labels_lengths, reduction,
    average_frames)`` without materialising the log-probabilities or their gradient.

    Args as ``ctct_loss`` (warp_ctct/__init__.py:88-112), with raw scores in place of
    log-probabilities: logits (N, T, U, V) float32 / float16 / bfloat16 on the GPU, V including
    the blank at index 0.  The gradient flows to ``logits`` (same shape and dtype).
    ``global_batch`` replaces N as the divisor of 'mean' (for a shard of a larger batch).
    """
    from . import _as_int, _reduce, _require_cuda
    assert average_frames is None or isinstance(average_frames, bool)
    assert reduction is None or reduction in ("none", "mean", "sum")
    assert logits.dim() == 4
    assert labels.dim() == 2
    assert logits.size(2) == labels.size(1) + 1
    assert logits.size(0) == labels.size(0) == frames_lengths.size(0) == labels_lengths.size(0)
    _require_cuda(log_probs=logits, ys=labels, lx=frames_lengths, ly=labels_lengths)
    enable_grad = logits.requires_grad and torch.is_grad_enabled()
    if logits.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        logits = logits.float()
    if not logits.is_contiguous():
        logits = logits.contiguous()
    ys, lx, ly = _as_int(labels), _as_int(frames_lengths), _as_int(labels_lengths)
    if reduction in ("mean", "sum") and logits.size(0) > 0:
        norm = float(logits.size(0) if global_batch is None else global_batch)
        return FusedLogitsCTCTLossReduced.apply(logits, ys, lx, ly, enable_grad, reduction == "mean",
                                                bool(average_frames), norm)
    costs = FusedLogitsCTCTLoss.apply(logits, ys, lx, ly, enable_grad)
    return _reduce(costs, frames_lengths, reduction, average_frames)
