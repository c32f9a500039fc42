"""Host-side logic of the batch-sharded driver: the shard planner and the global reduction,
exercised with world_size-2 gloo ranks on CPU (the costs themselves come from the GPU kernels
and are covered by the gpu tests)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from warp_ctct_b200 import sharded
from warp_ctct_b200.sharded import PendingLoss, plan_shards, reduce_costs, shard_weights


def _lengths(seed, G, lxr=(100, 400), lyr=(10, 100)):
    rng = np.random.default_rng(seed)
    lx = rng.integers(lxr[0], lxr[1] + 1, G)
    ly = np.minimum(rng.integers(lyr[0], lyr[1] + 1, G), lx // 2)
    return lx, ly


@pytest.mark.parametrize("G,world", [(256, 8), (256, 4), (64, 2), (37, 4), (5, 8), (32, 1)])
def test_plan_is_a_balanced_partition(G, world):
    lx, ly = _lengths(G + world, G)
    plan = plan_shards(lx, ly, world)
    assert len(plan) == world
    flat = sorted(i for p in plan for i in p)
    assert flat == list(range(G))
    counts = [len(p) for p in plan]
    assert max(counts) - min(counts) <= 1
    if G >= 8 * world:
        w = shard_weights(lx, ly, plan)
        assert max(w) / min(w) < 1.05, w
    assert plan == plan_shards(list(lx), list(ly), world)  # deterministic, accepts plain lists


def test_plan_beats_contiguous_split():
    lx, ly = _lengths(3, 256)
    order = np.argsort(lx)  # a length-sorted batch, the worst case for a contiguous split
    lx, ly = lx[order], ly[order]
    w_plan = shard_weights(lx, ly, plan_shards(lx, ly, 8))
    w_naive = shard_weights(lx, ly, [list(range(r * 32, (r + 1) * 32)) for r in range(8)])
    assert max(w_plan) / min(w_plan) < 1.05 < max(w_naive) / min(w_naive)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        G = 10
        lx = torch.arange(1, G + 1, dtype=torch.int32) + 4
        all_costs = torch.linspace(3.0, 30.0, G, dtype=torch.float32)
        plan = plan_shards(lx.tolist(), [2] * G, world)
        mine = torch.tensor(plan[rank])
        res = {}
        for red in ("mean", "sum"):
            for avg in (False, True):
                c = all_costs[mine].clone().requires_grad_(True)
                loss = reduce_costs(c, lx[mine], G, red, avg)
                loss.backward()
                ref = all_costs / lx if avg else all_costs
                want = ref.mean() if red == "mean" else ref.sum()
                scale = (1.0 / lx[mine] if avg else torch.ones(len(mine))) / (G if red == "mean" else 1)
                res[(red, avg)] = (abs(loss.item() - want.item()) < 1e-5 * abs(want.item()),
                                   torch.allclose(c.grad, scale.float(), rtol=1e-6))
        c = all_costs[mine].clone().requires_grad_(True)
        res["none"] = (torch.equal(reduce_costs(c, lx[mine], G, "none", False), c), True)
        # the all-reduce is asynchronous: backward() and metadata queries leave it in flight, the
        # first read of the value settles it
        c = all_costs[mine].clone().requires_grad_(True)
        loss = reduce_costs(c, lx[mine], G, "sum", False)
        pending = isinstance(loss, PendingLoss) and loss._work is not None
        shape_ok = loss.shape == () and loss.requires_grad and loss.dim() == 0
        still = loss._work is not None
        loss.backward()
        after_backward = loss._work is not None and torch.allclose(c.grad, torch.ones(len(mine)))
        doubled = loss * 2            # arithmetic reads the value: settles, returns a plain tensor
        settled = loss._work is None and type(doubled) is torch.Tensor
        value_ok = abs(doubled.item() - 2 * all_costs.sum().item()) < 1e-4 and abs(float(loss) - all_costs.sum().item()) < 1e-4
        res["pending"] = (pending and shape_ok and still and after_backward, settled and value_ok)
        # the queue of collectives in flight stays bounded: finished ones are dropped, and beyond the cap
        # the oldest is settled as a new one starts
        sharded._MAX_INFLIGHT = 4
        keep, longest = [], 0
        for _ in range(10):
            keep.append(reduce_costs(all_costs[mine].clone(), lx[mine], G, "mean", False))
            longest = max(longest, len(sharded._inflight))
        res["bounded"] = (longest <= 4, all(abs(k.item() - all_costs.mean().item()) < 1e-5 for k in keep))
        out[rank] = res
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_global_reduction_with_two_gloo_ranks():
    world = 2
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), out), nprocs=world, join=True)
        assert sorted(out.keys()) == [0, 1]
        for rank in range(world):
            for key, (ok_value, ok_grad) in out[rank].items():
                assert ok_value and ok_grad, (rank, key)


def test_nccl_entry_points_of_the_scalar_communicator_resolve():
    """The sharded loss on NCCL groups calls NCCL's C interface directly for its 4-byte all-reduce:
    the library torch runs on must offer those entry points, and the unique id must have nccl.h's size."""
    import ctypes

    assert ctypes.sizeof(sharded._NcclUniqueId) == 128
    lib = sharded._nccl_library()
    for name in ("ncclGetUniqueId", "ncclCommInitRank", "ncclAllReduce", "ncclCommDestroy", "ncclGetErrorString"):
        assert hasattr(lib, name), name
    version = ctypes.c_int()
    assert lib.ncclGetVersion(ctypes.byref(version)) == 0 and version.value >= 21800


def test_cpu_groups_keep_the_process_group_all_reduce():
    """No communicator of the library's own is made for a tensor that is not a float32 CUDA tensor."""
    buf = torch.zeros(())
    assert sharded._async_all_reduce(buf, None) is buf      # one rank: nothing to do
    assert not sharded._scalar_comms
