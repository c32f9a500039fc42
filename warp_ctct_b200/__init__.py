"""B200-native CTC-Transducer loss with the Python surface of maxwellzh/warp-ctct.

``ctct_loss`` and ``ctct_simple_loss`` keep the reference's signatures, assertions, reductions,
blank index (0) and autograd behaviour (warp_ctct/__init__.py:88-236).  Underneath, every step
runs in hand-written sm_100a CUDA kernels reached through the C ABI of ``libctct_b200.so``
(``include/ctct_b200.h``); there is no PyTorch, Triton or CPU fallback.

blank = 0
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from . import _lib

__version__ = "0.3.0"  # the reference release whose API this mirrors (setup.py:18)
__all__ = ["ctct_loss", "ctct_simple_loss"]  # as the reference; ctct_loss_and_grad is an extra

T = torch.Tensor


def _require_cuda(**tensors) -> None:
    # csrc/binding.cpp:14-16,44-49: every tensor argument must live on the GPU
    for name, t in tensors.items():
        if not t.is_cuda:
            raise RuntimeError(f"{name} must be located in the CUDA")


def _as_int(t: T) -> T:
    if t.dtype == torch.int32 and t.is_contiguous():
        return t
    return t.to(torch.int32).contiguous()


# The dense gradient is zero except for <= 3 columns per row, and clearing it needs nothing the
# forward pass computes.  With PREZERO on, the forward pass allocates the gradient and has it
# cleared by extra thread blocks of the (latency-bound) lattice launch; the backward pass then
# only patches the non-zero columns.  Off (or for small tensors, or on a second backward through
# the same graph) the backward pass writes the whole tensor in one pass.
# Set CTCT_B200_PREZERO=0 to turn it off.
PREZERO = os.environ.get("CTCT_B200_PREZERO", "1") != "0"
PREZERO_MIN_BYTES = 8 << 20
_ELEM_SIZE = {torch.float32: 4, torch.float16: 2, torch.bfloat16: 2}
_size_cache = {}


def _sizes(N: int, Tm: int, U1: int, want_grad: bool):
    """(bytes of the compact gradient rounded up to 256, workspace bytes), cached per shape."""
    key = (N, Tm, U1, want_grad)
    hit = _size_cache.get(key)
    if hit is None:
        lib = _lib.lib()
        ws = lib.ctct_b200_workspace_bytes(N, Tm, U1, int(want_grad))
        if ws == 0 and N > 0:
            raise RuntimeError(f"unsupported problem size N={N}, T={Tm}, U+1={U1}")
        g3 = (lib.ctct_b200_grads3_elems(N, Tm, U1) * 4 + 255) // 256 * 256 if want_grad else 0
        hit = _size_cache[key] = (g3, max(ws, 256))
    return hit


def _fused_forward(ctx, log_probs: T, labels: T, lx: T, ly: T, requires_grad: bool, red: int, average_frames: bool,
                   norm: float, device: Optional[torch.device] = None):
    """Shared forward of the two fused autograd functions: one C-ABI call (gather, lattice with the
    gradient buffer cleared on the side, occupancy gradient, optional reduction).
    Returns the float32 tensor [loss, costs[0..N)].  `device` is where everything but `log_probs`
    lives when `log_probs` itself is pinned host memory that the gather kernel reads in place."""
    N, Tm, U1, V = log_probs.shape
    dev = log_probs.device if device is None else device
    lib = _lib.lib()
    g3_bytes, ws_bytes = _sizes(N, Tm, U1, requires_grad)
    switch = torch.cuda.current_device() != dev.index
    if switch:
        prev = torch.cuda.current_device()
        torch.cuda.set_device(dev)
    try:
        out = torch.empty((N + 1,), dtype=torch.float32, device=dev)
        # one allocation: [compact gradient | workspace]; kept until the backward pass
        buf = torch.empty((g3_bytes + ws_bytes,), dtype=torch.uint8, device=dev)
        dense = None
        nbytes = N * Tm * U1 * V * _ELEM_SIZE[log_probs.dtype]
        if requires_grad and PREZERO and nbytes >= PREZERO_MIN_BYTES:
            dense = torch.empty((N, Tm, U1, V), dtype=log_probs.dtype, device=dev)
        base = buf.data_ptr()
        rc = lib.ctct_b200_loss_forward_fused(
            log_probs.data_ptr(), _lib.dtype_code(log_probs.dtype), labels.data_ptr(), lx.data_ptr(), ly.data_ptr(),
            N, Tm, U1, V, int(requires_grad), red, int(average_frames), norm, out.data_ptr() + 4, out.data_ptr(),
            base if requires_grad else None, dense.data_ptr() if dense is not None else None,
            nbytes if dense is not None else 0, base + g3_bytes, ws_bytes, torch._C._cuda_getCurrentRawStream(dev.index))
    finally:
        if switch:
            torch.cuda.set_device(prev)
    _lib.check(rc, "ctct_b200_loss_forward_fused")
    if requires_grad:
        ctx.save_for_backward(buf, labels, lx, ly)
        ctx.meta = (N, Tm, U1, V, log_probs.dtype, red, bool(average_frames), float(norm))
        ctx.cleared = dense
    return out


def _fused_backward(ctx, grad: T):
    """Shared backward: dense (N,T,U+1,V) gradient; `grad` is (N,) when red == 0, else a scalar."""
    buf, labels, lx, ly = ctx.saved_tensors
    N, Tm, U1, V, dtype, red, avg, norm = ctx.meta
    dev = buf.device
    lib = _lib.lib()
    go = grad.to(torch.float32).contiguous()
    dense, ctx.cleared = ctx.cleared, None
    switch = torch.cuda.current_device() != dev.index
    if switch:
        prev = torch.cuda.current_device()
        torch.cuda.set_device(dev)
    try:
        st = torch._C._cuda_getCurrentRawStream(dev.index)
        if dense is not None:  # cleared during the forward pass: patch the non-zero columns
            rc = lib.ctct_b200_loss_backward_patch(buf.data_ptr(), go.data_ptr(), int(red != 0), red, int(avg), norm,
                                                   labels.data_ptr(), lx.data_ptr(), ly.data_ptr(), N, Tm, U1, V,
                                                   _lib.dtype_code(dtype), dense.data_ptr(), st)
        else:
            dense = torch.empty((N, Tm, U1, V), dtype=dtype, device=dev)
            if red == 0:
                rc = lib.ctct_b200_loss_backward(buf.data_ptr(), go.data_ptr(), labels.data_ptr(), lx.data_ptr(),
                                                 ly.data_ptr(), N, Tm, U1, V, _lib.dtype_code(dtype), dense.data_ptr(), st)
            else:
                rc = lib.ctct_b200_loss_backward_reduced(buf.data_ptr(), go.data_ptr(), red, int(avg), norm,
                                                         labels.data_ptr(), lx.data_ptr(), ly.data_ptr(), N, Tm, U1, V,
                                                         _lib.dtype_code(dtype), dense.data_ptr(), st)
    finally:
        if switch:
            torch.cuda.set_device(prev)
    _lib.check(rc, "ctct_b200_loss_backward")
    return dense


class FusedCTCTLoss(torch.autograd.Function):
    """costs = CTC-T loss of the FULL joint tensor (N,T,U+1,V); gather, lattice and the
    occupancy gradient are fused behind one C-ABI call, the dense gradient behind another.

    Replaces the chain gather -> .float() -> CTCTLoss of warp_ctct/__init__.py:124-136."""

    @staticmethod
    def forward(ctx, log_probs: T, labels: T, lx: T, ly: T, requires_grad: bool):
        return _fused_forward(ctx, log_probs, labels, lx, ly, requires_grad, 0, False, 1.0)[1:]

    @staticmethod
    def backward(ctx, grad_outputs: T):
        return _fused_backward(ctx, grad_outputs), None, None, None, None


class FusedCTCTLossReduced(torch.autograd.Function):
    """FusedCTCTLoss with the reduction of warp_ctct/__init__.py:138-147 folded into the kernels:
    returns the 0-dim loss  sum_n costs[n] * w[n],  w[n] = (average_frames ? 1/lx[n] : 1) *
    (mean ? 1/norm : 1).  No separate sum / divide / expand kernels run in either direction."""

    @staticmethod
    def forward(ctx, log_probs: T, labels: T, lx: T, ly: T, requires_grad: bool, mean: bool, average_frames: bool,
                norm: float):
        return _fused_forward(ctx, log_probs, labels, lx, ly, requires_grad, 2 if mean else 1, bool(average_frames),
                              float(norm))[0]

    @staticmethod
    def backward(ctx, grad_loss: T):
        return _fused_backward(ctx, grad_loss), None, None, None, None, None, None, None


def ctct_loss_fwd(log_probs: T, ys: T, lx: T, ly: T, requires_grad: bool):
    """Extension-level entry point of the reference, ``_C.ctct_loss_fwd`` (csrc/binding.cpp:31-100):
    gathered float32 log-probs (N,T,U+1,3) -> (costs, grads); ``grads`` is ``costs`` when no
    gradient is requested.  Same checks, same error type."""
    for name, t in (("log_probs", log_probs), ("ys", ys), ("lx", lx), ("ly", ly)):
        if not t.is_contiguous():
            raise RuntimeError(f"{name} must be contiguous")
    if log_probs.dtype != torch.float32:
        raise RuntimeError("log_probs must be a Float tensor")
    for name, t in (("ys", ys), ("lx", lx), ("ly", ly)):
        if t.dtype != torch.int32:
            raise RuntimeError(f"{name} must be a Int tensor")
    _require_cuda(log_probs=log_probs, ys=ys, lx=lx, ly=ly)
    if log_probs.dim() != 4:
        raise RuntimeError("log probs must have 4 dims.")
    if log_probs.size(3) != 3:
        raise RuntimeError("log probs should be first gathered to length 3 at last dim.")
    if ys.dim() != 2:
        raise RuntimeError("targets must have 2 dims.")
    if lx.dim() != 1:
        raise RuntimeError("lx must have only 1 dim.")
    if ly.dim() != 1:
        raise RuntimeError("ly must have only 1 dim.")
    if not (log_probs.size(0) == ys.size(0) == lx.size(0) == ly.size(0)):
        raise RuntimeError("input args should match at dim 0 (batch N)")
    N, Tm, U1, _ = log_probs.shape
    dev = log_probs.device
    costs = torch.empty((N,), dtype=torch.float32, device=dev)
    grads = torch.empty_like(log_probs) if requires_grad else None
    with torch.cuda.device(dev):
        ws = _lib.workspace(N, Tm, U1, requires_grad, dev)
        rc = _lib.lib().ctct_b200_gathered_forward(
            _lib.ptr(log_probs), _lib.ptr(ys), _lib.ptr(lx), _lib.ptr(ly), N, Tm, U1, int(requires_grad),
            _lib.ptr(costs), _lib.ptr(grads), _lib.ptr(ws), ws.numel(), _lib.stream_ptr(dev))
    _lib.check(rc, "ctct_b200_gathered_forward")
    return (costs, grads) if requires_grad else (costs, costs)


class CTCTLoss(torch.autograd.Function):
    """Same contract as the reference class (warp_ctct/__init__.py:20-33): the input is the
    gathered (N,T,U+1,3) float32 tensor and the gradient has that shape."""

    @staticmethod
    def forward(ctx, log_probs: T, labels: T, lx: T, ly: T, requires_grad: bool):
        costs, grads = ctct_loss_fwd(log_probs, labels, lx, ly, requires_grad)
        if requires_grad:
            ctx.save_for_backward(grads)
        return costs

    @staticmethod
    def backward(ctx, grad_outputs: T):
        (grads,) = ctx.saved_tensors
        return grad_outputs.view(-1, 1, 1, 1) * grads, None, None, None, None


def _reduce(costs: T, frames_lengths: T, reduction, average_frames) -> T:
    # warp_ctct/__init__.py:138-147
    if average_frames:
        costs = costs / frames_lengths
    if reduction == "none" or reduction is None:
        return costs
    elif reduction == "sum":
        return costs.sum()
    elif reduction == "mean":
        return costs.mean()
    return costs


def ctct_loss(log_probs: torch.FloatTensor,
              labels: torch.IntTensor,
              frames_lengths: torch.IntTensor,
              labels_lengths: torch.IntTensor,
              reduction: Optional[str] = "mean",
              average_frames: bool = False) -> torch.Tensor:
    """The CTC-Transducer loss (drop-in for ``warp_ctct.ctct_loss``, warp_ctct/__init__.py:88-147).

    Args:
        log_probs: (N, T, U, V) log-probabilities; N batch, T frames, U = max labels + 1,
            V vocabulary including the blank at index 0.  float32, float16 or bfloat16
            (accumulation is float32); other floating types are converted to float32.
        labels: (N, U-1) integer labels.
        frames_lengths: (N,) number of frames per utterance.
        labels_lengths: (N,) number of labels per utterance.
        reduction: 'none' | 'mean' | 'sum' | None.
        average_frames: divide each utterance's loss by its number of frames.
    """
    assert average_frames is None or isinstance(average_frames, bool)
    assert reduction is None or reduction in ("none", "mean", "sum")

    assert log_probs.dim() == 4
    assert labels.dim() == 2
    assert log_probs.size(2) == labels.size(1) + 1
    assert log_probs.size(0) == labels.size(0) == frames_lengths.size(0) == labels_lengths.size(0)

    _require_cuda(log_probs=log_probs, ys=labels, lx=frames_lengths, ly=labels_lengths)
    enable_grad = log_probs.requires_grad and torch.is_grad_enabled()
    if log_probs.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        log_probs = log_probs.float()
    if not log_probs.is_contiguous():
        log_probs = log_probs.contiguous()
    if reduction in ("mean", "sum") and log_probs.size(0) > 0:
        return FusedCTCTLossReduced.apply(log_probs, _as_int(labels), _as_int(frames_lengths), _as_int(labels_lengths),
                                          enable_grad, reduction == "mean", bool(average_frames),
                                          float(log_probs.size(0)))
    costs = FusedCTCTLoss.apply(log_probs, _as_int(labels), _as_int(frames_lengths), _as_int(labels_lengths),
                                enable_grad)
    return _reduce(costs, frames_lengths, reduction, average_frames)


class _Saved:
    """Stand-in for an autograd context when forward and backward run back to back."""

    def save_for_backward(self, *tensors):
        self.saved_tensors = tensors


def ctct_loss_and_grad(log_probs: T, labels: T, frames_lengths: T, labels_lengths: T,
                       reduction: Optional[str] = "mean", average_frames: bool = False,
                       device: Optional[torch.device] = None, global_batch: Optional[int] = None):
    """Loss and its dense gradient d loss / d log_probs in one call (no counterpart in the reference,
    which always goes through autograd): for a loss that ends the graph, `loss.backward()` seeds 1.0,
    so both passes can run back to back.

    `log_probs` may live in PINNED HOST memory (e.g. a joint tensor that was off-loaded, or produced
    on the host): the gather kernel then reads the three log-probs it needs per (n, t, u) row in
    place over PCIe (about 100 bytes per row instead of V * sizeof), and nothing else touches the
    tensor.  Labels and lengths may be host tensors too (copied; they are tiny).  Loss and gradient
    are created on `device` (default: the device of `log_probs`, or the current CUDA device).

    Returns (loss, grad): `loss` as `ctct_loss` returns it, `grad` (N,T,U,V) in the dtype of
    `log_probs`; with reduction 'none' the gradient is that of `costs.sum()`.  `global_batch`
    replaces N as the divisor of 'mean' (for a shard of a larger batch)."""
    assert reduction is None or reduction in ("none", "mean", "sum")
    assert log_probs.dim() == 4 and labels.dim() == 2
    assert log_probs.size(2) == labels.size(1) + 1
    assert log_probs.size(0) == labels.size(0) == frames_lengths.size(0) == labels_lengths.size(0)
    if log_probs.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        raise RuntimeError("log_probs must be float32, float16 or bfloat16")
    if not log_probs.is_contiguous():
        raise RuntimeError("log_probs must be contiguous")
    if log_probs.is_cuda:
        dev = log_probs.device
    else:
        if not log_probs.is_pinned():
            raise RuntimeError("a host log_probs tensor must be in pinned memory (tensor.pin_memory())")
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    ys, lx, ly = (_as_int(t).to(dev, non_blocking=True) for t in (labels, frames_lengths, labels_lengths))
    N = log_probs.size(0)
    norm = float(N if global_batch is None else global_batch)
    red = {"mean": 2, "sum": 1}.get(reduction, 0)
    ctx = _Saved()
    out = _fused_forward(ctx, log_probs, ys, lx, ly, True, red, bool(average_frames) and red != 0, norm, device=dev)
    if red:
        seed = torch.ones((), dtype=torch.float32, device=dev)
        loss = out[0]
    else:
        seed = torch.ones((N,), dtype=torch.float32, device=dev)
        loss = out[1:]
        if average_frames:
            loss = loss / lx
            seed = seed / lx
    return loss, _fused_backward(ctx, seed)


from .logits import FusedLogitsCTCTLoss, FusedLogitsCTCTLossReduced, ctct_loss_from_logits  # noqa: E402,F401
from .packed import FusedPackedCTCTLoss, ctct_loss_packed, pack_joint, unpack_joint  # noqa: E402,F401
from .simple import (FusedSimpleCTCTLoss, LogMMExp, SimpleCTCTLoss, ctct_loss_simple_fwd,  # noqa: E402,F401
                     log_matmul, log_matmul_backward, log_matmul_tc)


def ctct_simple_loss(f: torch.FloatTensor,
                     g: torch.FloatTensor,
                     labels: torch.IntTensor,
                     frames_lengths: torch.IntTensor,
                     labels_lengths: torch.IntTensor,
                     reduction: Optional[str] = "mean",
                     average_frames: bool = False,
                     normalized: bool = True) -> torch.Tensor:
    """The CTC-Transducer loss with the log-add joiner (warp_ctct/__init__.py:150-236)."""
    from .simple import ctct_simple_loss as _impl

    return _impl(f, g, labels, frames_lengths, labels_lengths, reduction, average_frames, normalized)
