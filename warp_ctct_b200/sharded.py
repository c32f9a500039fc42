"""Batch-sharded CTC-T loss: one process per GPU, utterances split across ranks.

Utterances are independent in every kernel, so the data path needs no collective at all; the
only exchange is one all-reduce of the scalar sum of costs (4 bytes) so that every rank holds
the global loss.  The reference has no multi-GPU code; the reduction semantics are those of
warp_ctct/__init__.py:138-147 applied to the GLOBAL batch.
"""
from __future__ import annotations

import collections
import ctypes
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


# ---- the scalar all-reduce, kept off the compute stream -------------------------------------------
#
# The backward pass of a shard needs nothing from the other ranks: the gradient scale is the local
# utterance weight times the upstream gradient.  Only the VALUE of the reduced loss depends on the
# collective.  So the all-reduce is issued asynchronously (on a communication stream, ordered after
# the kernel that produced this rank's share: the library's own communicator on NCCL groups, see
# _ScalarComm, else the process group with async_op) and the compute stream waits for it only when
# somebody looks at the value: `loss.item()`, printing, arithmetic on it.
# `loss.backward()` does not, so the backward kernels of this step and the forward kernels of the
# next one run while the 4 bytes travel.

_NO_WAIT_NAMES = {"backward", "register_hook", "retain_grad", "size", "dim", "numel", "stride", "is_contiguous",
                  "requires_grad_", "__get__"}


class PendingLoss(torch.Tensor):
    """The reduced loss of a sharded step whose all-reduce may still be in flight.

    Behaves like the plain 0-dim tensor it wraps.  Any operation that reads the value first makes the
    current stream wait for the collective (`settle()`, idempotent; costs nothing once the
    collective is done); `backward()` and metadata queries do not."""

    _work = None

    def settle(self) -> None:
        work, self._work = self._work, None
        if work is not None:
            work.wait()   # stream wait for NCCL; host wait for gloo

    def backward(self, gradient=None, retain_graph=None, create_graph=False, inputs=None):
        # straight to autograd, without the detour through __torch_function__ (and without waiting)
        with torch._C.DisableTorchFunctionSubclass():
            return torch.Tensor.backward(self, gradient, retain_graph, create_graph, inputs)

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        if getattr(func, "__name__", "") not in _NO_WAIT_NAMES:
            for a in args:
                if isinstance(a, PendingLoss):
                    a.settle()
                elif isinstance(a, (list, tuple)):
                    for b in a:
                        if isinstance(b, PendingLoss):
                            b.settle()
        with torch._C.DisableTorchFunctionSubclass():
            return func(*args, **(kwargs or {}))


# Collectives in flight, as (handle, alias of the buffer): the buffers must stay alive until the
# communication stream is done with them.  A finished one is dropped after a look at its state from the host (no operation goes into the
# compute stream: a wait or a record between two kernels of the loss costs their programmatic overlap,
# a few microseconds each).  The host may run a few hundred kernels ahead of the GPU, so "still running"
# is the normal state of the newest entries; only when _MAX_INFLIGHT of them are, is the oldest one
# waited for on the stream, so that the queue stays bounded (a buffer is 4 bytes).
_inflight: collections.deque = collections.deque()
_MAX_INFLIGHT = 256


class _StreamWait:
    """What PendingLoss.settle() needs of a collective: wait() makes the current stream wait for it."""

    __slots__ = ("event", "device_index")

    def __init__(self, event, device_index):
        self.event = event
        self.device_index = device_index

    def is_completed(self) -> bool:
        return self.event.query()

    def wait(self):
        if torch.cuda.current_device() == self.device_index:
            self.event.wait()   # the current stream of the current device waits
        else:
            torch.cuda.current_stream(self.device_index).wait_event(self.event)


class _NcclUniqueId(ctypes.Structure):
    _fields_ = [("internal", ctypes.c_char * 128)]   # ncclUniqueId of nccl.h


def _nccl_library():
    """The NCCL shared library torch itself runs on (already loaded in this process), with the
    entry points of nccl.h this module calls."""
    lib = ctypes.CDLL("libnccl.so.2")
    lib.ncclGetErrorString.restype = ctypes.c_char_p
    lib.ncclGetErrorString.argtypes = [ctypes.c_int]
    lib.ncclGetUniqueId.argtypes = [ctypes.POINTER(_NcclUniqueId)]
    lib.ncclCommInitRank.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, _NcclUniqueId, ctypes.c_int]
    lib.ncclAllReduce.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int,
                                  ctypes.c_void_p, ctypes.c_void_p]
    lib.ncclCommDestroy.argtypes = [ctypes.c_void_p]
    return lib


_NCCL_FLOAT32, _NCCL_SUM = 7, 0   # ncclDataType_t / ncclRedOp_t of nccl.h


class _ScalarComm:
    """A communicator of this library's own for the one-float all-reduce of a CUDA process group.

    `torch.distributed.all_reduce` costs 50-100 microseconds of HOST time per call inside a step (work
    object, watchdog bookkeeping, argument checks, logging wrapper): about half of what it takes to
    enqueue the whole loss, and enough to make the sharded step host-bound.  The collective itself is
    four bytes.  So the first sharded call on an NCCL group creates an NCCL communicator over the same
    ranks through NCCL's C interface (the unique id travels through the process group once) and a
    communication stream, and every later call is: record an event on the compute stream, make the
    communication stream wait for it, ncclAllReduce there, record an event behind it."""

    def __init__(self, group, device):
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        uid = _NcclUniqueId()
        # Every rank must take the same road.  What can fail on one rank alone (loading the library,
        # making the id) happens first, and the ranks agree on the outcome through the process group
        # before any of them enters NCCL's own collective initialisation.
        failure = None
        try:
            self.lib = _nccl_library()
            if rank == 0:
                self._check(self.lib.ncclGetUniqueId(ctypes.byref(uid)), "ncclGetUniqueId")
        except Exception as exc:
            failure = exc
        ok = torch.tensor([0 if failure else 1], dtype=torch.int32, device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
        if int(ok.item()) == 0:
            raise RuntimeError(f"not available on every rank ({failure!r} here)")
        box = [ctypes.string_at(ctypes.addressof(uid), 128) if rank == 0 else None]
        dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        ctypes.memmove(ctypes.addressof(uid), box[0], 128)
        self.comm = ctypes.c_void_p()
        with torch.cuda.device(device):
            self._check(self.lib.ncclCommInitRank(ctypes.byref(self.comm), world, uid, rank), "ncclCommInitRank")
            self.stream = torch.cuda.Stream(device)
            # Events are recorded again and again instead of created per call.  A wait captures the
            # record that precedes it, so `ready` can be a single event.  The `done` events form a ring
            # longer than the queue of collectives in flight: the oldest one of the queue still has
            # its own record when it is looked at (waiting for it must not mean waiting for the newest
            # collective), and whoever holds a handle for longer than a lap waits for a later point of
            # the same stream, which implies its own.
            self.ready = torch.cuda.Event()
            index = torch.device(device).index
            self.done = [_StreamWait(torch.cuda.Event(), index) for _ in range(_MAX_INFLIGHT + 8)]
            self.turn = 0
        self.device_index = index
        self.stream_handle = ctypes.c_void_p(self.stream.cuda_stream)
        self.device = device

    def _check(self, rc: int, what: str) -> None:
        if rc != 0:
            raise RuntimeError(f"{what}: {self.lib.ncclGetErrorString(rc).decode()}")

    def all_reduce(self, buf: torch.Tensor) -> _StreamWait:
        assert buf.dtype == torch.float32 and buf.is_contiguous()
        if torch.cuda.current_device() == self.device_index:
            self.ready.record()   # on the current stream
        else:
            self.ready.record(torch.cuda.current_stream(self.device))
        self.stream.wait_event(self.ready)
        ptr = buf.data_ptr()
        self._check(self.lib.ncclAllReduce(ptr, ptr, buf.numel(), _NCCL_FLOAT32, _NCCL_SUM, self.comm, self.stream_handle),
                    "ncclAllReduce")
        done = self.done[self.turn]
        self.turn = (self.turn + 1) % len(self.done)
        done.event.record(self.stream)
        return done

    def close(self) -> None:
        if self.comm:
            self.stream.synchronize()
            self.lib.ncclCommDestroy(self.comm)
            self.comm = ctypes.c_void_p()


_scalar_comms: dict = {}
FAST_SCALAR_ALL_REDUCE = True   # False: always go through torch.distributed.all_reduce(async_op=True)


def _scalar_comm(group, device):
    """The _ScalarComm of (group, device), created on first use by ALL ranks of the group together;
    None when the group is not an NCCL group of CUDA devices (then torch.distributed does the job)."""
    pg = group if group is not None else dist.group.WORLD   # the default group is a new object after a re-init
    key = (id(pg), device.index)
    comm, owner = _scalar_comms.get(key, (False, None))
    if comm is False or owner is not pg:   # `owner` keeps the group object alive, so its id is not handed out again
        comm = None
        try:
            if FAST_SCALAR_ALL_REDUCE and device.type == "cuda" and "nccl" in str(dist.get_backend(group)):
                comm = _ScalarComm(group, device)
        except Exception as exc:   # e.g. no raw NCCL binding in this torch build: the process group still works
            import warnings
            warnings.warn(f"warp_ctct_b200: scalar communicator unavailable ({exc!r}); using torch.distributed.all_reduce")
            comm = None
        _scalar_comms[key] = (comm, pg)
    return comm


def close_scalar_comms() -> None:
    """Destroys the communicators this module created (every rank calls it, before
    torch.distributed.destroy_process_group); later sharded calls create new ones."""
    while _inflight:
        _inflight.popleft()[0].wait()
    for comm, _ in _scalar_comms.values():
        if comm is not None:
            comm.close()
    _scalar_comms.clear()


def _world_size(group) -> int:
    return dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1


def _start_all_reduce(buf: torch.Tensor, group, world: Optional[int] = None):
    """Starts the sum-all-reduce of `buf` in place.  Returns the handle of the collective (wait(),
    is_completed()), or None with one rank.  `world`: the size of the group where the caller has
    looked it up already."""
    if (world if world is not None else _world_size(group)) <= 1:
        return None
    comm = None
    if buf.is_cuda and buf.dtype == torch.float32 and buf.is_contiguous():
        comm = _scalar_comm(group, buf.device)
    if comm is not None:
        return comm.all_reduce(buf)
    return dist.all_reduce(buf, op=dist.ReduceOp.SUM, group=group, async_op=True)


def _pending(out: torch.Tensor, handle) -> torch.Tensor:
    """`out` (what autograd returned for the buffer whose all-reduce `handle` stands for) as a
    PendingLoss that owns the handle; enters it into the queue of collectives in flight."""
    if handle is None:
        return out
    queue = _inflight
    while queue and queue[0][0].is_completed():
        queue.popleft()
    # a detached alias keeps the storage alive without holding on to the autograd graph (and what it saved)
    queue.append((handle, out.detach()))
    while len(queue) > _MAX_INFLIGHT:
        queue.popleft()[0].wait()
    res = out.as_subclass(PendingLoss)
    res._work = handle
    return res


def _async_all_reduce(buf: torch.Tensor, group, world: Optional[int] = None) -> torch.Tensor:
    """Sum-all-reduce of `buf` in place, asynchronously: returns it as a PendingLoss (or as it is with one rank)."""
    return _pending(buf, _start_all_reduce(buf, group, world))


class _AllReduceSum(torch.autograd.Function):
    """y = sum over ranks of x.  Each rank back-propagates only through its own term, so the
    backward is the identity (every rank seeds the same global loss with the same grad)."""

    @staticmethod
    def forward(ctx, x: torch.Tensor, group):
        y = x.clone()
        _started.append(_start_all_reduce(y, group))
        return y

    @staticmethod
    def backward(ctx, grad):
        return grad, None


class _ShardedReducedLoss(torch.autograd.Function):
    """This rank's share of the reduced global loss straight out of the kernels (see
    FusedCTCTLossReduced), all-reduced in place: one 4-byte collective and no extra kernel.
    The backward is local and does not wait for the collective."""

    @staticmethod
    def forward(ctx, log_probs, labels, lx, ly, requires_grad: bool, mean: bool, average_frames: bool, norm: float,
                group, from_logits: bool, world: int):
        if from_logits:
            from .logits import _forward as fwd
            ctx.from_logits = True
            loss = fwd(ctx, log_probs, labels, lx, ly, requires_grad, 2 if mean else 1, bool(average_frames), float(norm))[0]
        else:
            ctx.from_logits = False
            loss = _fused_forward(ctx, log_probs, labels, lx, ly, requires_grad, 2 if mean else 1, bool(average_frames),
                                  float(norm))[0]
        _started.append(_start_all_reduce(loss, group, world))
        return loss

    @staticmethod
    def backward(ctx, grad_loss):
        if ctx.from_logits:
            from .logits import _backward as bwd
            return bwd(ctx, grad_loss), None, None, None, None, None, None, None, None, None, None
        return _fused_backward(ctx, grad_loss), None, None, None, None, None, None, None, None, None, None


# side channel from the forward of the two functions above to their caller: the handle of the collective
# that was started on the tensor they return (autograd hands back a new Python object for that tensor)
_started: list = []


def _attach(out: torch.Tensor) -> torch.Tensor:
    handle = _started.pop() if _started else None
    _started.clear()
    return _pending(out, handle)


def all_reduce_sum(x: torch.Tensor, group=None) -> torch.Tensor:
    return _attach(_AllReduceSum.apply(x, group))


def reduce_costs(costs: torch.Tensor, frames_lengths: torch.Tensor, global_batch: int, reduction: Optional[str],
                 average_frames: bool, group=None) -> torch.Tensor:
    """Reduction of warp_ctct/__init__.py:138-147 over the global batch from this rank's costs.
    The division of 'mean' is applied to the local sum, so that the all-reduce is the last operation
    and nothing on the compute stream waits for it."""
    if average_frames:
        costs = costs / frames_lengths
    if reduction == "none" or reduction is None:
        return costs  # per-utterance costs stay local
    share = costs.sum()
    if reduction == "mean":
        share = share / global_batch
    return all_reduce_sum(share, group)


def sharded_ctct_loss(log_probs: torch.Tensor, labels: torch.Tensor, frames_lengths: torch.Tensor,
                      labels_lengths: torch.Tensor, global_batch: Optional[int] = None,
                      reduction: Optional[str] = "mean", average_frames: bool = False, group=None,
                      from_logits: bool = False) -> torch.Tensor:
    """``ctct_loss`` on this rank's shard of a batch that is split across the process group.

    ``log_probs`` etc. hold only the local utterances.  With ``reduction`` 'mean' or 'sum' the
    returned scalar is the loss of the GLOBAL batch (identical on every rank) and its backward
    writes d(global loss)/d(local log_probs); 'none' returns the local per-utterance costs.
    ``global_batch`` defaults to the sum of local batch sizes when they are equal on all ranks.
    ``from_logits``: ``log_probs`` holds raw scores and the log-softmax is fused into the kernels
    (``ctct_loss_from_logits``).

    With more than one rank the scalar is a ``PendingLoss``: its all-reduce runs beside the
    backward pass, and the first operation that reads the value waits for it."""
    assert reduction is None or reduction in ("none", "mean", "sum")
    assert log_probs.dim() == 4 and labels.dim() == 2
    assert log_probs.size(2) == labels.size(1) + 1
    assert log_probs.size(0) == labels.size(0) == frames_lengths.size(0) == labels_lengths.size(0)
    _require_cuda(log_probs=log_probs, ys=labels, lx=frames_lengths, ly=labels_lengths)
    world = _world_size(group)
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
        return _attach(_ShardedReducedLoss.apply(log_probs, _as_int(labels), _as_int(frames_lengths),
                                                 _as_int(labels_lengths), enable_grad, reduction == "mean",
                                                 bool(average_frames), float(global_batch), group, bool(from_logits), world))
    if from_logits:
        from .logits import FusedLogitsCTCTLoss
        costs = FusedLogitsCTCTLoss.apply(log_probs, _as_int(labels), _as_int(frames_lengths), _as_int(labels_lengths),
                                          enable_grad)
    else:
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
    world = _world_size(group)
    if global_batch is None:
        global_batch = f.size(0) * world
    track_f = f.requires_grad and torch.is_grad_enabled()
    track_g = g.requires_grad and torch.is_grad_enabled()
    costs = FusedSimpleCTCTLoss.apply(f.float().contiguous(), g.float().contiguous(), _as_int(labels),
                                      _as_int(frames_lengths), _as_int(labels_lengths), bool(normalized),
                                      track_f, track_g)
    return reduce_costs(costs, frames_lengths, global_batch, reduction, bool(average_frames), group)
