"""CTC-Transducer loss on a PACKED joint tensor: only the valid rows of every utterance exist.

The reference pads every utterance to (T, U+1) rows; its kernels skip the padding
(csrc/gather.cu:321) but the tensor, and the gradient autograd builds for it
(warp_ctct/__init__.py:124-131), still carry it: 30-70 % of all bytes for ragged batches.
Here the joint tensor is (rows, V) with rows = sum_n frames[n] * (labels[n] + 1); utterance n owns a
contiguous block, frame-major, labels[n] + 1 rows per frame.  The gradient has the same packed
shape.  ``from_logits`` selects the variant with the log-softmax fused in.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib

T = torch.Tensor


def valid_mask(frames_lengths: T, labels_lengths: T, max_frames: int, max_contexts: int) -> T:
    """(N, max_frames, max_contexts) boolean mask of the rows a packed tensor keeps."""
    dev = frames_lengths.device
    t = torch.arange(max_frames, device=dev).view(1, -1, 1)
    u = torch.arange(max_contexts, device=dev).view(1, 1, -1)
    return (t < frames_lengths.view(-1, 1, 1)) & (u <= labels_lengths.view(-1, 1, 1))


def pack_joint(x: T, frames_lengths: T, labels_lengths: T) -> T:
    """(N,T,U,V) padded -> (rows, V) packed (a copy)."""
    return x[valid_mask(frames_lengths, labels_lengths, x.size(1), x.size(2))]


def unpack_joint(packed: T, frames_lengths: T, labels_lengths: T, max_frames: int, max_contexts: int) -> T:
    """(rows, V) packed -> (N,T,U,V) padded with zeros."""
    out = packed.new_zeros((frames_lengths.numel(), max_frames, max_contexts, packed.size(1)))
    out[valid_mask(frames_lengths, labels_lengths, max_frames, max_contexts)] = packed
    return out


class FusedPackedCTCTLoss(torch.autograd.Function):
    """The reduced loss (red = 1 'sum', 2 'mean') or the per-utterance costs (red = 0) from a packed
    joint tensor; gradient of the same packed shape."""

    @staticmethod
    def forward(ctx, packed: T, labels: T, lx: T, ly: T, requires_grad: bool, red: int, average_frames: bool, norm: float,
                max_frames: int, from_logits: bool):
        from . import _sizes
        N, U1 = labels.size(0), labels.size(1) + 1
        R, V = packed.shape
        dev = packed.device
        lib = _lib.lib()
        g3_bytes, ws_bytes = _sizes(N, max_frames, U1, requires_grad)
        esize = packed.element_size()
        with _lib.on_device(dev):
            st = _lib.raw_stream(dev)
            out = torch.empty((N + 1,), dtype=torch.float32, device=dev)
            cu = torch.empty((N + 1,), dtype=torch.int64, device=dev)
            _lib.check(lib.ctct_b200_packed_offsets(lx.data_ptr(), ly.data_ptr(), N, max_frames, U1, cu.data_ptr(), st),
                       "ctct_b200_packed_offsets")
            buf = torch.empty((g3_bytes + ws_bytes,), dtype=torch.uint8, device=dev)
            base = buf.data_ptr()
            grad = None
            common = (packed.data_ptr(), _lib.dtype_code(packed.dtype), cu.data_ptr(), R, labels.data_ptr(), lx.data_ptr(),
                      ly.data_ptr(), N, max_frames, U1, V, int(requires_grad), red, int(average_frames), norm,
                      out.data_ptr() + 4, out.data_ptr(), base if requires_grad else None)
            if from_logits:
                rc = lib.ctct_b200_logits_forward_packed(*common, base + g3_bytes, ws_bytes, st)
            else:
                if requires_grad:   # cleared by extra blocks of the lattice launch, patched in the backward pass
                    grad = torch.empty_like(packed)
                rc = lib.ctct_b200_loss_forward_packed(*common, _lib.ptr(grad), R * V * esize if grad is not None else 0,
                                                       base + g3_bytes, ws_bytes, st)
        _lib.check(rc, "ctct_b200_*_forward_packed")
        if requires_grad:
            ctx.save_for_backward(buf, packed, cu, labels, lx, ly)
            ctx.meta = (N, max_frames, U1, V, R, red, bool(average_frames), float(norm), bool(from_logits))
            ctx.cleared = grad
        return out[0] if red else out[1:]

    @staticmethod
    def backward(ctx, grad_out: T):
        buf, packed, cu, labels, lx, ly = ctx.saved_tensors
        N, Tm, U1, V, R, red, avg, norm, from_logits = ctx.meta
        dev = packed.device
        lib = _lib.lib()
        go = grad_out.to(torch.float32).contiguous()   # one float for a reduced loss, else N
        out, ctx.cleared = ctx.cleared, None
        with _lib.on_device(dev):
            st = _lib.raw_stream(dev)
            if from_logits:
                out = torch.empty_like(packed)
                rc = lib.ctct_b200_logits_backward_packed(
                    buf.data_ptr(), go.data_ptr(), int(red != 0), red, int(avg), norm, packed.data_ptr(), cu.data_ptr(), R,
                    labels.data_ptr(), lx.data_ptr(), ly.data_ptr(), N, Tm, U1, V, _lib.dtype_code(packed.dtype),
                    out.data_ptr(), st)
            else:
                if out is None:   # second backward through a retained graph: clear a fresh buffer first
                    out = torch.empty_like(packed)
                    _lib.check(lib.ctct_b200_zero_fill(out.data_ptr(), out.numel() * out.element_size(), st), "zero_fill")
                rc = lib.ctct_b200_loss_backward_packed(
                    buf.data_ptr(), go.data_ptr(), int(red != 0), red, int(avg), norm, cu.data_ptr(), R, labels.data_ptr(),
                    lx.data_ptr(), ly.data_ptr(), N, Tm, U1, V, _lib.dtype_code(packed.dtype), out.data_ptr(), st)
        _lib.check(rc, "ctct_b200_*_backward_packed")
        return out, None, None, None, None, None, None, None, None, None


def ctct_loss_packed(log_probs: T, labels: T, frames_lengths: T, labels_lengths: T, reduction: Optional[str] = "mean",
                     average_frames: bool = False, max_frames: Optional[int] = None, from_logits: bool = False,
                     global_batch: Optional[int] = None) -> T:
    """``ctct_loss`` (warp_ctct/__init__.py:88-147) for a packed joint tensor.

    Args:
        log_probs: (rows, V) log-probabilities (raw scores with ``from_logits``) of the valid rows only,
            rows = sum_n frames_lengths[n] * (labels_lengths[n] + 1), utterance after utterance,
            frame-major inside an utterance; float32 / float16 / bfloat16, contiguous, on the GPU.
        labels: (N, U) padded labels;  frames_lengths, labels_lengths: (N,).
        max_frames: an upper bound of frames_lengths known on the host; omitted, it is read back from
            the device (one synchronisation, as the reference's own size query, csrc/binding.cpp:68).
    The gradient flows to ``log_probs`` and has its packed shape.  Lengths that do not add up to
    ``rows`` are not detected; rows they would place beyond the tensor are not touched.
    """
    from . import _as_int, _require_cuda
    assert average_frames is None or isinstance(average_frames, bool)
    assert reduction is None or reduction in ("none", "mean", "sum")
    assert log_probs.dim() == 2 and labels.dim() == 2
    assert labels.size(0) == frames_lengths.size(0) == labels_lengths.size(0)
    _require_cuda(log_probs=log_probs, ys=labels, lx=frames_lengths, ly=labels_lengths)
    if log_probs.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        log_probs = log_probs.float()
    if not log_probs.is_contiguous():
        log_probs = log_probs.contiguous()
    if max_frames is None:
        max_frames = int(frames_lengths.max().item()) if frames_lengths.numel() else 0
    N = labels.size(0)
    enable_grad = log_probs.requires_grad and torch.is_grad_enabled()
    red = {"mean": 2, "sum": 1}.get(reduction, 0)
    norm = float(max(N, 1) if global_batch is None else global_batch)
    lx = _as_int(frames_lengths)
    out = FusedPackedCTCTLoss.apply(log_probs, _as_int(labels), lx, _as_int(labels_lengths), enable_grad, red,
                                    bool(average_frames) and red != 0, norm, int(max_frames), bool(from_logits))
    if red:
        return out
    return out / frames_lengths if average_frames else out
