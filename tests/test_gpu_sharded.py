"""The batch-sharded loss on real GPUs: two ranks, one process per GPU, NCCL.  Checks that the shards
add up to the single-process loss on the whole batch (value and gradient), that the scalar all-reduce
goes through the library's own communicator and stays pending across backward(), and that many steps
without reading the loss neither pile up nor change the values.  Needs two GPUs (skipped otherwise)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from util import make_case

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank(rank, world, port, out):
    import warp_ctct_b200 as W
    from warp_ctct_b200 import sharded
    from warp_ctct_b200.sharded import PendingLoss, plan_shards, sharded_ctct_loss

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    res = {}
    try:
        G, T, U1, V = 8 * world, 64, 17, 512
        lp, ys, lx, ly = make_case(G, T, U1, V, 1.5, 77, lx_range=(30, 64), ly_range=(3, 16), cap_half=True)
        mine = np.array(plan_shards(lx, ly, world)[rank])
        d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
        for from_logits in (False, True):
            xa = d(lp).requires_grad_(True)      # the whole batch on this GPU
            ref = (W.ctct_loss_from_logits if from_logits else W.ctct_loss)(xa, d(ys), d(lx), d(ly), reduction="mean")
            ref.backward()
            x = d(lp[mine]).requires_grad_(True)
            loss = sharded_ctct_loss(x, d(ys[mine]), d(lx[mine]), d(ly[mine]), global_batch=G, reduction="mean",
                                     from_logits=from_logits)
            pending = isinstance(loss, PendingLoss) and loss._work is not None
            loss.backward()
            still = loss._work is not None        # backward() does not wait for the collective
            value = loss.item()
            settled = loss._work is None
            res[f"value from_logits={from_logits}"] = abs(value - ref.item()) < 1e-5 * abs(ref.item())
            res[f"grad from_logits={from_logits}"] = (x.grad - xa.grad[mine]).abs().max().item() < 1e-6
            res[f"pending from_logits={from_logits}"] = pending and still and settled
        res["own communicator"] = any(isinstance(c, sharded._ScalarComm) for c, _ in sharded._scalar_comms.values())
        losses = []
        for _ in range(300):                       # more steps than the event ring is long
            x = d(lp[mine]).requires_grad_(True)
            step_loss = sharded_ctct_loss(x, d(ys[mine]), d(lx[mine]), d(ly[mine]), global_batch=G, reduction="mean")
            step_loss.backward()
            losses.append(step_loss)
        values = [v.item() for v in losses]
        res["unread steps"] = (max(values) - min(values) < 1e-6 * abs(values[0])
                               and abs(values[0] - ref.item()) < 1e-5 * abs(ref.item())
                               and len(sharded._inflight) <= sharded._MAX_INFLIGHT)
        out[rank] = res
    finally:
        dist.barrier()
        sharded.close_scalar_comms()
        dist.destroy_process_group()


@pytest.mark.timeout(600)
def test_two_ranks_add_up_to_the_whole_batch():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_rank, args=(world, _free_port(), out), nprocs=world, join=True)
        assert sorted(out.keys()) == [0, 1]
        for rank in range(world):
            for key, ok in out[rank].items():
                assert ok, (rank, key)
