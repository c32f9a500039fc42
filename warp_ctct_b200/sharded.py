"""Batch-sharded CTC-T loss: one process per GPU, utterances split across ranks.

Utterances are independent in every kernel, so the data path needs no collective at all; the
only exchange is one all-reduce of the scalar sum of costs (4 bytes) so that every rank holds
the global loss.  The reference has no multi-GPU code; the reduction semantics are those of
warp_ctct/__init__.py:138-147 applied to the GLOBAL batch.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from . import FusedCTCTLoss, _as_int, _fused_backward, _fused_forward, _require_cuda


def plan_shards(frames_lengths: Sequence[int], labels_lengths: Sequence[int], world_size: int) -> List[List[int]]:
    """Length-balanced assignment of utterances to ranks.

    Work per utterance is proportional to lx * (ly + 1) (gathered rows, lattice cells and patched
    gradient rows).  Utterances are sorted by that weight and dealt in a snake (0..G-1, G-1..0, ...)
    so that every rank gets the same COUNT (+-1) and nearly the same total weight.  Deterministic,
    so every rank can compute the same plan from the same lengths without communication."""
    lx = [int(v) for v in frames_lengths]
    ly = [int(v) for v in labels_lengths]
    assert len(lx) == len(ly) and world_size >= 1
    order = sorted(range(len(lx)), key=lambda n: (-(lx[n] * (ly[n] + 1)), n))
    plan: List[List[int]] = [[] for _ in range(world_size)]
    for pos, n in enumerate(order):
        lap, k = divmod(pos, world_size)
        plan[k if lap % 2 == 0 else world_size - 1 - k].append(n)
    return plan


def shard_weights(frames_lengths, labels_lengths, plan) -> List[int]:
    return [sum(int(frames_lengths[n]) * (int(labels_lengths[n]) + 1) for n in idx) for idx in plan]


def _multi_rank(group) -> bool:
    return dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1


class _AllReduceSum(torch.autograd.Function):
    """y = sum over ranks of x.  Each rank back-propagates only through its own term, so the
    backward is the identity (every rank seeds the same global loss with the same grad)."""

    @staticmethod
    def forward(ctx, x: torch.Tensor, group):
        y = x.clone()
        if _multi_rank(group):
            dist.all_reduce(y, op=dist.ReduceOp.SUM, group=group)
        return y

    @staticmethod
    def backward(ctx, grad):
        return grad, None


class _ShardedReducedLoss(torch.autograd.Function):
    """This rank's share of the reduced global loss straight out of the kernels (see
    FusedCTCTLossReduced), all-reduced in place before autograd ever sees it: one 4-byte
    collective and no extra kernel.  The backward is local."""

    @staticmethod
    def forward(ctx, log_probs, labels, lx, ly, requires_grad: bool, mean: bool, average_frames: bool, norm: float,
                group):
        loss = _fused_forward(ctx, log_probs, labels, lx, ly, requires_grad, 2 if mean else 1, bool(average_frames),
                              float(norm))[0]
        if _multi_rank(group):
            dist.all_reduce(loss, op=dist.ReduceOp.SUM, group=group)
        return loss

    @staticmethod
    def backward(ctx, grad_loss):
        return _fused_backward(ctx, grad_loss), None, None, None, None, None, None, None, None


def all_reduce_sum(x: torch.Tensor, group=None) -> torch.Tensor:
    return _AllReduceSum.apply(x, group)


def reduce_costs(costs: torch.Tensor, frames_lengths: torch.Tensor, global_batch: int, reduction: Optional[str],
                 average_frames: bool, group=None) -> torch.Tensor:
    """Reduction of warp_ctct/__init__.py:138-147 over the global batch from this rank's costs."""
    if average_frames:
        costs = costs / frames_lengths
    if reduction == "none" or reduction is None:
        return costs  # per-utterance costs stay local
    total = all_reduce_sum(costs.sum(), group)
    if reduction == "mean":
        return total / global_batch
    return total


def sharded_ctct_loss(log_probs: torch.Tensor, labels: torch.Tensor, frames_lengths: torch.Tensor,
                      labels_lengths: torch.Tensor, global_batch: Optional[int] = None,
                      reduction: Optional[str] = "mean", average_frames: bool = False, group=None) -> torch.Tensor:
    """``ctct_loss`` on this rank's shard of a batch that is split across the process group.

    ``log_probs`` etc. hold only the local utterances.  With ``reduction`` 'mean' or 'sum' the
    returned scalar is the loss of the GLOBAL batch (identical on every rank) and its backward
    writes d(global loss)/d(local log_probs); 'none' returns the local per-utterance costs.
    ``global_batch`` defaults to the sum of local batch sizes when they are equal on all ranks."""
    assert reduction is None or reduction in ("none", "mean", "sum")
    assert log_probs.dim() == 4 and labels.dim() == 2
    assert log_probs.size(2) == labels.size(1) + 1
    assert log_probs.size(0) == labels.size(0) == frames_lengths.size(0) == labels_lengths.size(0)
    _require_cuda(log_probs=log_probs, ys=labels, lx=frames_lengths, ly=labels_lengths)
    world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
    if global_batch is None:
        global_batch = log_probs.size(0) * world
    enable_grad = log_probs.requires_grad and torch.is_grad_enabled()
    if log_probs.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        log_probs = log_probs.float()
    if not log_probs.is_contiguous():
        log_probs = log_probs.contiguous()
    if reduction in ("mean", "sum") and log_probs.size(0) > 0:
        # this rank's share of the global loss straight out of the kernels (for 'mean' already
        # divided by the global batch); the all-reduce of that one float completes it
        return _ShardedReducedLoss.apply(log_probs, _as_int(labels), _as_int(frames_lengths), _as_int(labels_lengths),
                                         enable_grad, reduction == "mean", bool(average_frames), float(global_batch),
                                         group)
    costs = FusedCTCTLoss.apply(log_probs, _as_int(labels), _as_int(frames_lengths), _as_int(labels_lengths),
                                enable_grad)
    return reduce_costs(costs, frames_lengths, global_batch, reduction, average_frames, group)


def sharded_ctct_simple_loss(f: torch.Tensor, g: torch.Tensor, labels: torch.Tensor, frames_lengths: torch.Tensor,
                             labels_lengths: torch.Tensor, global_batch: Optional[int] = None,
                             reduction: Optional[str] = "mean", average_frames: bool = False,
                             normalized: bool = True, group=None) -> torch.Tensor:
    """``ctct_simple_loss`` (log-add joiner, warp_ctct/__init__.py:150-236) on this rank's shard of a
    batch split across the process group; reductions as in ``sharded_ctct_loss``."""
    from .simple import FusedSimpleCTCTLoss

    assert reduction is None or reduction in ("none", "mean", "sum")
    assert f.dim() == 3 and g.dim() == 3 and labels.dim() == 2
    assert g.size(1) == labels.size(1) + 1
    assert f.size(0) == g.size(0) == labels.size(0) == frames_lengths.size(0) == labels_lengths.size(0)
    _require_cuda(f=f, g=g, ys=labels, lx=frames_lengths, ly=labels_lengths)
    world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
    if global_batch is None:
        global_batch = f.size(0) * world
    track_f = f.requires_grad and torch.is_grad_enabled()
    track_g = g.requires_grad and torch.is_grad_enabled()
    costs = FusedSimpleCTCTLoss.apply(f.float().contiguous(), g.float().contiguous(), _as_int(labels),
                                      _as_int(frames_lengths), _as_int(labels_lengths), bool(normalized),
                                      track_f, track_g)
    return reduce_costs(costs, frames_lengths, global_batch, reduction, bool(average_frames), group)
