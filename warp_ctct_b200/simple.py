"""CTC-Transducer loss with the log-add joiner (``ctct_simple_loss``) and the reference's
auxiliary autograd classes, on the sm_100a kernels behind the C ABI.

Mirrors warp_ctct/__init__.py:36-85 (LogMMExp, SimpleCTCTLoss) and :150-236 (ctct_simple_loss).
"""
from __future__ import annotations

from typing import Any, Optional

import torch

from . import _lib

T = torch.Tensor


def _require_cuda(**tensors) -> None:
    for name, t in tensors.items():
        if not t.is_cuda:
            raise RuntimeError(f"{name} must be located in the CUDA")


# --------------------------------------------------------------------------------------------
# extension-level entry points of the reference (module warp_ctct._C, csrc/binding.cpp:326-345)

def log_matmul(lhs: T, rhs: T) -> T:
    """res[b,i,j] = log sum_k exp(lhs[b,i,k] + rhs[b,k,j]); float32, any strides
    (``_C.log_matmul``, csrc/binding.cpp:224-245)."""
    if lhs.dtype != torch.float32:
        raise RuntimeError("self must be a Float tensor")
    if rhs.dtype != torch.float32:
        raise RuntimeError("other must be a Float tensor")
    if not lhs.is_cuda:
        raise RuntimeError("need cuda tensors")
    if lhs.device != rhs.device:
        raise RuntimeError("need tensors on same GPU")
    if lhs.dim() != 3 or rhs.dim() != 3 or lhs.size(2) != rhs.size(1):
        raise RuntimeError("invalid sizes")
    B, M, K = lhs.shape
    N = rhs.size(2)
    # the result has the batch of lhs; rhs is expanded to it (csrc/logmatmul.cu:148-167), so a
    # batch of one on the right broadcasts (batch stride 0) and anything else must match
    if rhs.size(0) != B and rhs.size(0) != 1:
        raise RuntimeError(f"The expanded size of the tensor ({B}) must match the existing size ({rhs.size(0)}) at "
                           f"non-singleton dimension 0")
    rhs_sb = rhs.stride(0) if rhs.size(0) == B else 0
    out = torch.empty((B, M, N), dtype=torch.float32, device=lhs.device)
    with torch.cuda.device(lhs.device):
        rc = _lib.lib().ctct_b200_log_matmul(
            _lib.ptr(lhs), lhs.stride(0), lhs.stride(1), lhs.stride(2),
            _lib.ptr(rhs), rhs_sb, rhs.stride(1), rhs.stride(2),
            B, M, K, N, _lib.ptr(out), _lib.stream_ptr(lhs.device))
    _lib.check(rc, "ctct_b200_log_matmul")
    return out


def log_matmul_tc(f: T, g: T, keep_workspace: bool = False):
    """den[b,i,j] = log sum_k exp(f[b,i,k] + g[b,j,k]) for contiguous float32 f (B,M,K), g (B,N,K):
    the tensor-core path (tcgen05 GEMM on max-shifted exponentials, log/max epilogue) when the
    shape allows it (K % 8 == 0, K >= 64), otherwise the exact kernel.  Same values as
    ``log_matmul(f, g.transpose(1, 2))`` to float32 rounding.  With ``keep_workspace`` returns
    (den, workspace): the workspace (None on the exact path) holds the operand planes that the
    tensor-core backward pass of the simple loss reuses."""
    B, M, K = f.shape
    N = g.size(1)
    lib = _lib.lib()
    nbytes = lib.ctct_b200_log_matmul_tc_workspace_bytes(B, M, N, K)
    if nbytes == 0 or not (f.is_contiguous() and g.is_contiguous()) or f.data_ptr() % 16 or g.data_ptr() % 16:
        den = log_matmul(f, g.transpose(1, 2))
        return (den, None) if keep_workspace else den
    dev = f.device
    den = torch.empty((B, M, N), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        ws = torch.empty((nbytes,), dtype=torch.uint8, device=dev)
        rc = lib.ctct_b200_log_matmul_tc(f.data_ptr(), g.data_ptr(), B, M, N, K, den.data_ptr(), ws.data_ptr(), nbytes,
                                         _lib.stream_ptr(dev))
    _lib.check(rc, "ctct_b200_log_matmul_tc")
    return (den, ws) if keep_workspace else den


def log_matmul_backward(grad_out: Optional[T], lhs: T, rhs: T, res: T, grad_masks):
    """(grad_lhs, grad_rhs) of ``log_matmul`` for any (signed) ``grad_out``
    (``_C.log_matmul_backward``, csrc/binding.cpp:247-324)."""
    if grad_out is None:
        return None, None
    B, M, K = lhs.shape
    N = rhs.size(2)
    dev = lhs.device
    lhs_c = lhs.contiguous()
    broadcast_rhs = rhs.size(0) == 1 and B > 1   # undone below by a sum over the batch (csrc/binding.cpp:285-292)
    if broadcast_rhs:
        rhs = rhs.expand(B, -1, -1)
    rhs_t = rhs.transpose(1, 2).contiguous()  # (B,N,K); free when rhs is a transposed view
    go = grad_out.to(torch.float32).contiguous()
    res_c = res.contiguous()
    grad_lhs = torch.empty((B, M, K), dtype=torch.float32, device=dev) if grad_masks[0] else None
    grad_rhs_t = torch.empty((B, N, K), dtype=torch.float32, device=dev) if grad_masks[1] else None
    with torch.cuda.device(dev):
        rc = _lib.lib().ctct_b200_log_matmul_backward(
            _lib.ptr(go), _lib.ptr(lhs_c), _lib.ptr(rhs_t), _lib.ptr(res_c), B, M, K, N,
            _lib.ptr(grad_lhs), _lib.ptr(grad_rhs_t), _lib.stream_ptr(dev))
    _lib.check(rc, "ctct_b200_log_matmul_backward")
    if grad_rhs_t is not None and broadcast_rhs:
        grad_rhs_t = grad_rhs_t.sum(0, keepdim=True)
    return grad_lhs, (grad_rhs_t.transpose(1, 2) if grad_rhs_t is not None else None)


def _tc_operands(lhs: T, rhs: T):
    """(f, g) = (lhs, rhs^T) when they are what the tensor-core kernels take: float32 CUDA tensors,
    lhs (B,M,K) contiguous and rhs (B,K,N) a transposed view of a contiguous (B,N,K) tensor (what
    warp_ctct/__init__.py:199 passes), 16-byte aligned, K % 8 == 0, K >= 64; else None."""
    if not (lhs.is_cuda and rhs.is_cuda and lhs.dtype == torch.float32 and rhs.dtype == torch.float32):
        return None
    if lhs.dim() != 3 or rhs.dim() != 3 or lhs.size(0) != rhs.size(0) or lhs.size(2) != rhs.size(1):
        return None
    g = rhs.transpose(1, 2)
    if not (lhs.is_contiguous() and g.is_contiguous()) or lhs.data_ptr() % 16 or g.data_ptr() % 16:
        return None
    B, M, K = lhs.shape
    if _lib.lib().ctct_b200_log_matmul_tc_workspace_bytes(B, M, g.size(1), K) == 0:
        return None
    return lhs, g


class LogMMExp(torch.autograd.Function):
    """log(exp(lhs) @ exp(rhs)) with its analytic backward (warp_ctct/__init__.py:36-52).  Runs on
    the tensor cores, forward and backward, when the operands allow it (see _tc_operands)."""

    @staticmethod
    def forward(ctx: Any, lhs: T, rhs: T, track_l: bool = True, track_r: bool = True) -> T:
        ops = _tc_operands(lhs, rhs)
        if ops is not None:
            mm, ws = log_matmul_tc(ops[0], ops[1], keep_workspace=True)
        else:
            mm, ws = log_matmul(lhs, rhs), None
        if track_l or track_r:
            ctx.save_for_backward(lhs, rhs, mm, ws if ws is not None else lhs.new_empty(0))
            ctx.track = [track_l, track_r]
        return mm

    @staticmethod
    def backward(ctx: Any, grad_outputs: T) -> Any:
        lhs, rhs, res, ws = ctx.saved_tensors
        if ws.numel() == 0:
            grad_lhs, grad_rhs = log_matmul_backward(grad_outputs, lhs, rhs, res, ctx.track)
            return grad_lhs, grad_rhs, None, None
        B, M, K = lhs.shape
        g = rhs.transpose(1, 2)  # contiguous (B,N,K)
        N = g.size(1)
        dev = lhs.device
        go = grad_outputs.to(torch.float32).contiguous()
        grad_lhs = torch.empty((B, M, K), dtype=torch.float32, device=dev) if ctx.track[0] else None
        grad_g = torch.empty((B, N, K), dtype=torch.float32, device=dev) if ctx.track[1] else None
        with torch.cuda.device(dev):
            rc = _lib.lib().ctct_b200_log_matmul_backward_tc(
                _lib.ptr(go), _lib.ptr(lhs), _lib.ptr(g), _lib.ptr(res), B, M, K, N, _lib.ptr(grad_lhs), _lib.ptr(grad_g),
                _lib.ptr(ws), ws.numel(), _lib.stream_ptr(dev))
        _lib.check(rc, "ctct_b200_log_matmul_backward_tc")
        return grad_lhs, (grad_g.transpose(1, 2) if grad_g is not None else None), None, None


# --------------------------------------------------------------------------------------------
# fused loss on the full f and g

class FusedSimpleCTCTLoss(torch.autograd.Function):
    """costs of the log-add-joiner loss from the FULL f (N,T,V) and g (N,U+1,V).

    Forward: denominator (if normalised), then one C-ABI call that gathers, composes
    f + g - den, runs the lattice and the occupancy gradient.  Backward: one C-ABI call that
    writes the dense grad_f and grad_g (lattice part + the part through the denominator).
    Replaces LogMMExp + the two gathers + SimpleCTCTLoss of warp_ctct/__init__.py:195-225."""

    @staticmethod
    def forward(ctx, f: T, g: T, labels: T, lx: T, ly: T, normalized: bool, track_f: bool, track_g: bool):
        N, Tm, V = f.shape
        U1 = g.size(1)
        dev = f.device
        lib = _lib.lib()
        want_grad = track_f or track_g
        den, tc_ws = (log_matmul_tc(f, g, keep_workspace=True) if normalized else (None, None))
        if not want_grad:
            tc_ws = None
        costs = torch.empty((N,), dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            ws = _lib.workspace(N, Tm, U1, want_grad, dev)
            grads3 = None
            if want_grad:
                grads3 = torch.empty((lib.ctct_b200_grads3_elems(N, Tm, U1),), dtype=torch.float32, device=dev)
            rc = lib.ctct_b200_simple_forward(
                _lib.ptr(f), _lib.ptr(g), _lib.ptr(den), _lib.ptr(labels), _lib.ptr(lx), _lib.ptr(ly),
                N, Tm, U1, V, int(want_grad), _lib.ptr(costs), _lib.ptr(grads3), _lib.ptr(ws), ws.numel(),
                _lib.stream_ptr(dev))
        _lib.check(rc, "ctct_b200_simple_forward")
        if want_grad:
            ctx.save_for_backward(grads3, f, g, den if den is not None else f.new_empty(0), labels, lx, ly,
                                  tc_ws if tc_ws is not None else f.new_empty(0))
            ctx.meta = (N, Tm, U1, V, normalized, track_f, track_g)
        return costs

    @staticmethod
    def backward(ctx, grad_outputs: T):
        grads3, f, g, den, labels, lx, ly, tc_ws = ctx.saved_tensors
        N, Tm, U1, V, normalized, track_f, track_g = ctx.meta
        dev = f.device
        go = grad_outputs.to(torch.float32).contiguous()
        grad_f = torch.empty((N, Tm, V), dtype=torch.float32, device=dev) if track_f else None
        grad_g = torch.empty((N, U1, V), dtype=torch.float32, device=dev) if track_g else None
        with torch.cuda.device(dev):
            if normalized and tc_ws.numel() > 0:
                # gradient through the denominator as tensor-core GEMMs on the forward pass's planes
                rc = _lib.lib().ctct_b200_simple_backward_tc(
                    _lib.ptr(grads3), _lib.ptr(go), _lib.ptr(f), _lib.ptr(g), _lib.ptr(den),
                    _lib.ptr(labels), _lib.ptr(lx), _lib.ptr(ly), N, Tm, U1, V, _lib.ptr(grad_f), _lib.ptr(grad_g),
                    _lib.ptr(tc_ws), tc_ws.numel(), _lib.stream_ptr(dev))
            else:
                rc = _lib.lib().ctct_b200_simple_backward(
                    _lib.ptr(grads3), _lib.ptr(go), _lib.ptr(f), _lib.ptr(g), _lib.ptr(den) if normalized else None,
                    _lib.ptr(labels), _lib.ptr(lx), _lib.ptr(ly), N, Tm, U1, V, _lib.ptr(grad_f), _lib.ptr(grad_g),
                    _lib.stream_ptr(dev))
        _lib.check(rc, "ctct_b200_simple_backward")
        return grad_f, grad_g, None, None, None, None, None, None


def ctct_loss_simple_fwd(f: T, g: T, ys: T, den: T, lx: T, ly: T, requires_grad: bool):
    """``_C.ctct_loss_simple_fwd`` of the reference (csrc/binding.cpp:103-222): pre-gathered
    f (N,T,U+1), g (N,U+1,3), optional den (N,T,U+1; anything that is not 3-D means "none")
    -> (costs, grad_f, grad_g, grad_den) with the reference's shapes; gradients are None
    when ``requires_grad`` is false."""
    for name, t in (("f", f), ("g", g), ("ys", ys), ("lx", lx), ("ly", ly)):
        if not t.is_contiguous():
            raise RuntimeError(f"{name} must be contiguous")
    for name, t in (("f", f), ("g", g)):
        if t.dtype != torch.float32:
            raise RuntimeError(f"{name} must be a Float tensor")
    for name, t in (("ys", ys), ("lx", lx), ("ly", ly)):
        if t.dtype != torch.int32:
            raise RuntimeError(f"{name} must be a Int tensor")
    _require_cuda(f=f, g=g, ys=ys, lx=lx, ly=ly)
    if f.dim() != 3:
        raise RuntimeError("f must have 3 dims.")
    if g.dim() != 3:
        raise RuntimeError("g must have 3 dims.")
    if f.size(2) != g.size(1):
        raise RuntimeError("f should be gathered at last dim to length U matching the g at dim 1.")
    if g.size(2) != 3:
        raise RuntimeError("g should be first gathered to length 3 at last dim.")
    if ys.dim() != 2:
        raise RuntimeError("targets must have 2 dims.")
    if lx.dim() != 1:
        raise RuntimeError("lx must have only 1 dim.")
    if ly.dim() != 1:
        raise RuntimeError("ly must have only 1 dim.")
    if not (f.size(0) == g.size(0) == ys.size(0) == lx.size(0) == ly.size(0)):
        raise RuntimeError("input args should match at dim 0 (batch N)")
    normalized = den is not None and den.dim() == 3
    if normalized:
        if not den.is_contiguous():
            raise RuntimeError("den must be contiguous")
        _require_cuda(den=den)
        if den.dtype != torch.float32:
            raise RuntimeError("den must be a Float tensor")
    # compose f + g - den (csrc/simple.cu:20-26), lattice, occupancy gradient and the reductions of
    # csrc/binding.cpp:198,209-219: one C-ABI call, all CUDA
    N, Tm, U1 = f.shape
    dev = f.device
    lib = _lib.lib()
    costs = torch.empty((N,), dtype=torch.float32, device=dev)
    grad_f = torch.empty_like(f) if requires_grad else None
    grad_g = torch.empty_like(g) if requires_grad else None
    grad_den = torch.empty_like(den) if (requires_grad and normalized) else None
    with torch.cuda.device(dev):
        nbytes = lib.ctct_b200_simple_gathered_workspace_bytes(N, Tm, U1, int(requires_grad))
        if nbytes == 0 and N > 0:
            raise RuntimeError(f"unsupported problem size N={N}, T={Tm}, U+1={U1}")
        ws = torch.empty((max(nbytes, 256),), dtype=torch.uint8, device=dev)
        rc = lib.ctct_b200_simple_gathered_forward(
            _lib.ptr(f), _lib.ptr(g), _lib.ptr(den) if normalized else None, _lib.ptr(ys), _lib.ptr(lx), _lib.ptr(ly),
            N, Tm, U1, int(requires_grad), _lib.ptr(costs), _lib.ptr(grad_f), _lib.ptr(grad_g), _lib.ptr(grad_den),
            _lib.ptr(ws), ws.numel(), _lib.stream_ptr(dev))
    _lib.check(rc, "ctct_b200_simple_gathered_forward")
    return costs, grad_f, grad_g, grad_den


class SimpleCTCTLoss(torch.autograd.Function):
    """Same contract as the reference class (warp_ctct/__init__.py:55-85): pre-gathered f, g
    and an optional denominator; gradients w.r.t. those three."""

    @staticmethod
    def forward(ctx, f: T, g: T, den: Optional[T], labels: T, lx: T, ly: T, rg_f: bool, rg_g: bool):
        costs, grad_f, grad_g, grad_den = ctct_loss_simple_fwd(f, g, labels, den, lx, ly, (rg_f or rg_g))
        if not rg_f:
            grad_f = None
        if not rg_g:
            grad_g = None
        if not (den is not None and den.dim() == 3 and (rg_f or rg_g)):
            grad_den = None
        ctx.save_for_backward(grad_f, grad_g, grad_den)
        return costs

    @staticmethod
    def backward(ctx, grad_outputs: T):
        grad_f, grad_g, grad_den = ctx.saved_tensors
        grad_outputs = grad_outputs.view(-1, 1, 1)
        if grad_f is not None:
            grad_f = grad_f * grad_outputs
        if grad_g is not None:
            grad_g = grad_g * grad_outputs
        if grad_den is not None:
            grad_den = grad_den * grad_outputs
        return grad_f, grad_g, grad_den, None, None, None, None, None


def ctct_simple_loss(f, g, labels, frames_lengths, labels_lengths, reduction="mean", average_frames=False,
                     normalized=True) -> torch.Tensor:
    """Drop-in for ``warp_ctct.ctct_simple_loss`` (warp_ctct/__init__.py:150-236).

    Args:
        f: (N, T, V) acoustic scores;  g: (N, U, V) label-context scores, U = max labels + 1.
        labels: (N, U-1);  frames_lengths, labels_lengths: (N,).
        normalized: subtract log sum_v exp(f + g) (log-softmax of the joint) when True.
    """
    from . import _as_int, _reduce

    assert average_frames is None or isinstance(average_frames, bool)
    assert reduction is None or reduction in ("none", "mean", "sum")

    assert f.dim() == 3 and g.dim() == 3
    assert labels.dim() == 2
    assert g.size(1) == labels.size(1) + 1
    assert f.size(0) == g.size(0) == labels.size(0) == frames_lengths.size(0) == labels_lengths.size(0)

    _require_cuda(f=f, g=g, ys=labels, lx=frames_lengths, ly=labels_lengths)
    track_f = f.requires_grad and torch.is_grad_enabled()
    track_g = g.requires_grad and torch.is_grad_enabled()
    # the kernels compute in float32 (the reference calls .float() on both, :196-197,218)
    costs = FusedSimpleCTCTLoss.apply(f.float().contiguous(), g.float().contiguous(), _as_int(labels),
                                      _as_int(frames_lengths), _as_int(labels_lengths), bool(normalized),
                                      track_f, track_g)
    return _reduce(costs, frames_lengths, reduction, average_frames)
