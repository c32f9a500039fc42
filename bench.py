#!/usr/bin/env python
"""Benchmark of the CTC-Transducer loss hot path (fwd + bwd of ctct_loss) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload c2|c3|c5]

One "step" is one forward + backward of ``ctct_loss`` over one batch of synthetic utterances per
GPU.  Default workload (``c2``): float32 log-probs = log_softmax(1.5 * N(0,1)), B=32 per GPU,
T=256, U+1=65, V=512, frame lengths U[128,256], label lengths U[16,64] capped at frames/2.
With N > 1 (launched by torchrun, one rank per GPU) a global batch of 32*N utterances is
split length-balanced over the ranks; the only collective is the scalar-loss all-reduce.

Prints ONE JSON line (rank 0).  ``--impl reference`` times the CPU restatement of the
reference's algorithm (oracle/) on the host cores instead.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (B per GPU, T, U+1, V, dtype, sigma, lx range, ly range, cap ly at lx//2)
    "c2": (32, 256, 65, 512, "f32", 1.5, (128, 256), (16, 64), True),
    "c3": (16, 512, 129, 1024, "f16", 2.0, (256, 512), (32, 128), False),
    "c5": (32, 400, 101, 1024, "f16", 2.0, (100, 400), (10, 100), True),
}
# ctct_simple_loss (log-add joiner): (B per GPU, T, U+1, V, lx range, ly range); f, g ~ N(0,1) fp32
SIMPLE_WORKLOADS = {
    "c4": (32, 500, 101, 4096, (250, 500), (25, 100)),
    "c4s": (16, 500, 101, 4096, (250, 500), (25, 100)),   # small case of the same kernels for ncu captures
}
METRIC = "utterances/sec fwd+bwd"
UNIT = "utt/s"

# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of one launch of the dominant kernel, from the
# ncu captures summarised in profiles/: c2 = the lattice launch with its clearing blocks
# (ctct_loss_c2_kernels.md); c4 = the fused backward kernel of the denominator, captured at half the
# batch (c4s, simple_loss_c4s_kernels.md) and doubled, since traffic is proportional to the number
# of utterances.
NCU_TRAFFIC_PER_LAUNCH = {"c2": 10796544 + 1038705000, "c4s": 187469824 + 113467392,
                          "c4": 2 * (187469824 + 113467392)}


def workload_string(name, n_gpus):
    B, T, U1, V, dt, sigma, lxr, lyr, cap = WORKLOADS[name]
    return (f"{name}: ctct_loss {dt} fwd+bwd, B={B}/GPU (global {B * n_gpus}), T={T}, U+1={U1}, V={V}, "
            f"log_softmax({sigma}*N(0,1)), lx~U{list(lxr)}, ly~U{list(lyr)}" + (" capped lx//2" if cap else ""))


def global_lengths(name, n_gpus, seed=2000):
    if name in SIMPLE_WORKLOADS:
        B, T, U1, V, lxr, lyr = SIMPLE_WORKLOADS[name]
        cap = False
    else:
        B, T, U1, V, dt, sigma, lxr, lyr, cap = WORKLOADS[name]
    rng = np.random.default_rng(seed)
    G = B * n_gpus
    lx = rng.integers(lxr[0], lxr[1] + 1, G).astype(np.int32)
    ly = rng.integers(lyr[0], lyr[1] + 1, G).astype(np.int32)
    if cap:
        ly = np.minimum(ly, lx // 2).astype(np.int32)
    ly = np.minimum(ly, lx).astype(np.int32)
    ys = rng.integers(1, V, (G, U1 - 1)).astype(np.int32)
    return lx, ly, ys


def peaks(key="hbm_gbs", fallback=6650.0):
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            return float(json.load(fh)[key]), "measured"
    except Exception:
        return fallback, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    def __init__(self, device_index: int, period_s: float = 0.01):
        super().__init__(daemon=True)
        self.period, self.samples, self.reasons, self.stop_flag = period_s, [], set(), threading.Event()
        self.max_mhz, self.ok = None, False
        try:
            import pynvml
            import torch
            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            uuid = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
            try:
                self.h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            self.nv = pynvml
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self.ok = True
        except Exception:
            self.ok = False

    def sample(self):
        nv = self.nv
        self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
        mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)) if hasattr(
            nv, "nvmlDeviceGetCurrentClocksEventReasons") else int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
        names = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
                 0x80: "hw_power_brake_slowdown"}
        for bit, name in names.items():
            if mask & bit:
                self.reasons.add(name)

    def run(self):
        if not self.ok:
            return
        while not self.stop_flag.is_set():
            try:
                self.sample()
            except Exception:
                break
            time.sleep(self.period)

    def finish(self):
        self.stop_flag.set()
        if self.is_alive():
            self.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# --------------------------------------------------------------------------------------- reference arm

def run_reference(args):
    """CPU arm: the C restatement of the reference's algorithm (oracle/) on all host threads."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    import oracle
    B, T, U1, V, dt, sigma, lxr, lyr, cap = WORKLOADS[args.workload]
    lx, ly, ys = global_lengths(args.workload, 1)
    rng = np.random.default_rng(2000)
    x = sigma * rng.standard_normal((B, T, U1, V), dtype=np.float32)
    x -= x.max(-1, keepdims=True)
    lp = x - np.log(np.exp(x).sum(-1, keepdims=True))
    if dt == "f16":
        lp = lp.astype(np.float16).astype(np.float32)
    go = np.full((B,), 1.0 / B, np.float32)
    cores = oracle.max_threads()
    for _ in range(args.warmup):
        oracle.ctct_loss(lp, ys, lx, ly, go, nthreads=cores)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.ctct_loss(lp, ys, lx, ly, go, nthreads=cores)
    dt_s = time.perf_counter() - t0
    value = B * args.steps / dt_s
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt_s / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dt, "data": "synthetic",
        "config": {"workload": workload_string(args.workload, 1)},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"every step = the full batch of {B} utterances on {cores} OpenMP threads"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))
    return 0


# --------------------------------------------------------------------------------------- B200 arm

def setup_device(args):
    """One process per GPU: picks the device, brings up NCCL under torchrun.  Returns (world, rank, local_rank, dev)."""
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
        args.gpus = world
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the CTC-T kernels have no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        # NCCL announces its version on stdout when the communicator comes up; keep stdout for the JSON line
        sys.stdout.flush()
        saved = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=dev)
            dist.all_reduce(torch.zeros(1, device=dev))
            torch.cuda.synchronize(dev)
        finally:
            sys.stdout.flush()
            os.dup2(saved, 1)
            os.close(saved)
    return world, rank, local_rank, dev


def run_b200(args):
    import torch
    import torch.distributed as dist

    import warp_ctct_b200 as W
    from warp_ctct_b200 import _lib
    from warp_ctct_b200.sharded import plan_shards, sharded_ctct_loss, shard_weights

    world, rank, local_rank, dev = setup_device(args)
    lib = _lib.lib()

    B, T, U1, V, dt, sigma, lxr, lyr, cap = WORKLOADS[args.workload]
    tdt = {"f32": torch.float32, "f16": torch.float16}[dt]
    esize = {"f32": 4, "f16": 2}[dt]
    lx_g, ly_g, ys_g = global_lengths(args.workload, world)
    plan = plan_shards(lx_g, ly_g, world)
    mine = np.array(plan[rank])
    lx, ly, ys = lx_g[mine], ly_g[mine], ys_g[mine]
    assert len(mine) == B

    gen = torch.Generator(device=dev).manual_seed(2000 + rank)
    lp = (sigma * torch.randn((B, T, U1, V), device=dev, generator=gen)).log_softmax(-1).to(tdt)
    lp.requires_grad_(True)
    ys_t = torch.from_numpy(ys).to(dev)
    lx_t = torch.from_numpy(lx).to(dev)
    ly_t = torch.from_numpy(ly).to(dev)
    G = B * world

    def step():
        lp.grad = None
        loss = sharded_ctct_loss(lp, ys_t, lx_t, ly_t, global_batch=G, reduction="mean")
        loss.backward()
        return loss

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()

    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed_pass():
        """K steps between two events (barrier + synchronize on both sides), max over ranks."""
        barrier()
        ev0.record()
        t_host = time.perf_counter()
        for _ in range(args.steps):
            out = step()
        enqueue_us = 1e6 * (time.perf_counter() - t_host) / args.steps  # host time to enqueue one step
        ev1.record()
        barrier()
        t = torch.tensor([ev0.elapsed_time(ev1)], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()), enqueue_us, out

    # the timed region: nothing but the K steps
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    ms_total, host_us, loss = timed_pass()
    clocks = sampler.finish() if sampler else None

    # the same K steps once more with the library recording CUDA events around its kernels (the
    # event records between dependent launches cost a few microseconds per step, so this pass is
    # kept out of `value`): per-kernel durations for the roofline
    cap_n = 3 * args.steps + 3
    _lib.check(lib.ctct_b200_profile_enable(cap_n), "profile_enable")
    ms_profiled, _, _ = timed_pass()
    buf = np.zeros((cap_n, 4), np.float32)
    kinds = np.zeros((cap_n,), np.int32)
    n_rec = lib.ctct_b200_profile_read(buf.ctypes.data, kinds.ctypes.data, cap_n)
    lib.ctct_b200_profile_disable()
    fwd = buf[:n_rec][kinds[:n_rec] == 0]
    bwd = buf[:n_rec][kinds[:n_rec] == 1]
    # with PREZERO the lattice launch also clears the dense gradient (extra thread blocks) and the
    # backward pass only patches it; otherwise the backward pass writes the gradient in one pass
    precleared = bool(W.PREZERO) and B * T * U1 * V * esize >= W.PREZERO_MIN_BYTES
    k_ms = {"gather": float(fwd[:, 0].mean()), "lattice": float(fwd[:, 1].mean()),
            "fill_grad": float(fwd[:, 2].mean())}
    if precleared:
        k_ms["dense_patch"] = float(bwd[:, 0].mean())
    else:
        k_ms["dense_grad"] = float(bwd[:, 0].mean())
    dense_key = "lattice" if precleared else "dense_grad"

    value = G * args.steps / (ms_total * 1e-3)
    peak, peak_kind = peaks()
    rows_valid = int((lx.astype(np.int64) * (ly + 1)).sum())
    dense_bytes = B * T * U1 * V * esize + rows_valid * 16  # written once + compact gradient records read
    gather_bytes = rows_valid * 3 * 32 + B * T * U1 * 16    # one 32-byte sector per picked element + records out
    if precleared:
        dense_bytes = B * T * U1 * V * esize
    ach = dense_bytes / (k_ms[dense_key] * 1e-3) / 1e9
    roofline = {"kernel": ("k_lattice, clearing role (dense gradient streamer; shares the launch with the lattice CTAs)"
                           if precleared else "k_dense_grad (dense gradient streamer)"), "bound": "hbm", "achieved": ach, "peak": peak,
                "unit": "GB/s", "frac": ach / peak, "peak_source": f"of {peak_kind}",
                "algorithmic_bytes": dense_bytes, "traffic": NCU_TRAFFIC_PER_LAUNCH.get(args.workload)}
    g_ach = gather_bytes / (k_ms["gather"] * 1e-3) / 1e9
    kernels = {
        "gather": {"ms": k_ms["gather"], "sector_bytes": gather_bytes, "GB/s": g_ach, "frac": g_ach / peak},
        "fill_grad": {"ms": k_ms["fill_grad"]},
        "sum_ms": sum(k_ms.values()),
    }
    if precleared:
        kernels["lattice_and_clear"] = {"ms": k_ms["lattice"], "GB/s": ach, "frac": ach / peak,
                                        "note": "one launch: 2 lattice CTAs per utterance + blocks that zero the gradient"}
        kernels["dense_patch"] = {"ms": k_ms["dense_patch"]}
        # the lattice recursion by itself: a few steps with the clearing moved out of its launch
        # (one-pass dense gradient in the backward pass), event recording on
        W.PREZERO = False
        try:
            n_alone = 10
            _lib.check(lib.ctct_b200_profile_enable(3 * n_alone), "profile_enable")
            for _ in range(n_alone):
                step()
            torch.cuda.synchronize(dev)
            buf2 = np.zeros((3 * n_alone, 4), np.float32)
            kinds2 = np.zeros((3 * n_alone,), np.int32)
            n2 = lib.ctct_b200_profile_read(buf2.ctypes.data, kinds2.ctypes.data, 3 * n_alone)
            lib.ctct_b200_profile_disable()
            alone = buf2[:n2][kinds2[:n2] == 0][:, 1]
            rows = max(int(lx.max()), 1)
            kernels["lattice_alone"] = {"ms": float(alone.mean()), "ns_per_row": 1e6 * float(alone.mean()) / rows,
                                        "note": "alpha and beta CTAs of all utterances run concurrently; rows = frames of "
                                                "the longest utterance; measured with the clearing blocks taken out"}
        finally:
            W.PREZERO = True
    else:
        kernels["lattice"] = {"ms": k_ms["lattice"], "ns_per_row": 1e6 * k_ms["lattice"] / max(int(lx.max()), 1),
                              "note": "alpha and beta CTAs of all utterances run concurrently; rows = longest utterance"}
        kernels["dense_grad"] = {"ms": k_ms["dense_grad"], "GB/s": ach, "frac": ach / peak}

    # ---- the same step captured once in a CUDA graph and replayed (single GPU; informational) ----
    graph_ms = None
    if world == 1:
        try:
            # a fresh leaf over the same memory: its gradient accumulator must belong to the capturing stream
            lp_g = lp.detach().requires_grad_(True)

            def graph_step():
                sharded_ctct_loss(lp_g, ys_t, lx_t, ly_t, global_batch=G, reduction="mean").backward()

            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(2):
                    lp_g.grad = None
                    graph_step()
            torch.cuda.current_stream().wait_stream(side)
            lp_g.grad = None
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                graph_step()
            for _ in range(3):
                graph.replay()
            torch.cuda.synchronize(dev)
            ev0.record()
            for _ in range(args.steps):
                graph.replay()
            ev1.record()
            torch.cuda.synchronize(dev)
            graph_ms = ev0.elapsed_time(ev1) / args.steps
            del graph, lp_g
        except Exception as exc:  # capture is an extra: report why it did not happen
            graph_ms = f"not captured: {exc}"
        lp.grad = None

    # ---- end to end through the public API, inputs in pinned host memory ----
    e2e_steps = max(1, min(args.steps, args.e2e_steps))
    lp_host = torch.empty((B, T, U1, V), dtype=tdt, pin_memory=True)
    lp_host.copy_(lp.detach())
    ys_h, lx_h, ly_h = ys_t.cpu().pin_memory(), lx_t.cpu().pin_memory(), ly_t.cpu().pin_memory()
    del lp
    torch.cuda.empty_cache()

    def e2e_copy_step():
        # the whole joint tensor crosses PCIe, then the usual autograd path
        x = lp_host.to(dev, non_blocking=True).requires_grad_(True)
        y, a, b = ys_h.to(dev, non_blocking=True), lx_h.to(dev, non_blocking=True), ly_h.to(dev, non_blocking=True)
        loss = sharded_ctct_loss(x, y, a, b, global_batch=G, reduction="mean")
        loss.backward()
        return float(loss.item())  # device -> host read of the step's result

    def e2e_step():
        # the joint tensor stays in pinned host memory: the gather kernel reads the three log-probs it
        # needs per row in place over PCIe; labels and lengths are copied; loss read back
        loss, grad = W.ctct_loss_and_grad(lp_host, ys_h, lx_h, ly_h, reduction="mean", device=dev, global_batch=G)
        if world > 1:
            dist.all_reduce(loss)
        return float(loss.item())

    def timed(fn, n):
        for _ in range(2):
            fn()
        barrier()
        ev0.record()
        for _ in range(n):
            fn()
        ev1.record()
        barrier()
        t = torch.tensor([ev0.elapsed_time(ev1)], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    ms_e = timed(e2e_step, e2e_steps)
    ms_c = timed(e2e_copy_step, e2e_steps)
    small = ys_h.numel() * 4 + lx_h.numel() * 4 + ly_h.numel() * 4
    # one 32-byte sector per picked element (host-resident tensors are read without a fill-size hint)
    h2d = rows_valid * 3 * 32 + small
    e2e = {"value": G * e2e_steps / (ms_e * 1e-3), "unit": UNIT, "h2d_bytes_per_step": int(h2d * world),
           "d2h_bytes_per_step": 4 * world, "steps": e2e_steps,
           "note": "ctct_loss_and_grad on the joint tensor in pinned host memory: the gather kernel reads the 3 "
                   "log-probs per valid row in place over PCIe (one 32-byte sector each), labels and lengths are copied, "
                   "the dense gradient stays on the device, the loss scalar is read back",
           "full_copy": {"value": G * e2e_steps / (ms_c * 1e-3), "unit": UNIT,
                         "h2d_bytes_per_step": int((lp_host.numel() * esize + small) * world),
                         "note": "same step with the whole joint tensor copied host to device first (autograd path)"}}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_total / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": dt, "data": "synthetic",
        "config": {"workload": workload_string(args.workload, world),
                   "l2": f"inputs larger than L2: {B * T * U1 * V * esize / 1e9:.2f} GB joint tensor read sparsely and "
                         f"an equally large gradient written every step (L2 is 126 MB)",
                   "shard_weights": shard_weights(lx_g, ly_g, plan)},
        "clocks": clocks, "e2e": e2e, "gpu_launches": 4 * args.steps * world,
        "roofline": roofline, "kernels": kernels, "host_enqueue_us_per_step": host_us,
        "profiled_pass_ms_per_step": ms_profiled / args.steps,
    }
    if graph_ms is not None:
        line["cuda_graph_replay_ms_per_step"] = graph_ms

    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        import oracle
        cores = oracle.max_threads()
        lp_np = lp_host.float().numpy()
        go = np.full((B,), 1.0 / B, np.float32)
        oracle.ctct_loss(lp_np, ys, lx, ly, go, nthreads=cores)
        reps, t0 = 3, time.perf_counter()
        for _ in range(reps):
            costs_cpu, _ = oracle.ctct_loss(lp_np, ys, lx, ly, go, nthreads=cores)
        dt_s = (time.perf_counter() - t0) / reps
        line["cpu_baseline"] = {"value": B / dt_s, "unit": UNIT, "cores": cores, "kind": "port",
                                "sample": f"the full batch of {B} utterances, mean of {reps} passes, "
                                          f"{cores} OpenMP threads; loss agrees with the GPU to "
                                          f"{abs(float(costs_cpu.mean()) - float(loss.item())) / float(costs_cpu.mean()):.1e} rel"}
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


# --------------------------------------------------------------------------------------- ctct_simple_loss (c4)

def simple_inputs_host(name, seed=2000):
    B, T, U1, V, lxr, lyr = SIMPLE_WORKLOADS[name]
    rng = np.random.default_rng(seed)
    f = rng.standard_normal((B, T, V), dtype=np.float32)
    g = rng.standard_normal((B, U1, V), dtype=np.float32)
    return f, g


def simple_workload_string(name, n_gpus):
    B, T, U1, V, lxr, lyr = SIMPLE_WORKLOADS[name]
    return (f"{name}: ctct_simple_loss f32 fwd+bwd (normalized), B={B}/GPU (global {B * n_gpus}), T={T}, U+1={U1}, "
            f"V={V}, f,g~N(0,1), lx~U{list(lxr)}, ly~U{list(lyr)}")


def run_reference_simple(args):
    """CPU arm for the log-add-joiner loss: the C restatement on all host threads, on a bounded
    sample of the batch (the first utterances) so that a run ends within minutes."""
    if int(os.environ.get("RANK", "0")) != 0:
        return 0
    import oracle
    B, T, U1, V, lxr, lyr = SIMPLE_WORKLOADS[args.workload]
    lx, ly, ys = global_lengths(args.workload, 1)
    f, g = simple_inputs_host(args.workload)
    nb = min(B, 4)
    cores = oracle.max_threads()
    go = np.full((nb,), 1.0 / B, np.float32)

    def one():
        return oracle.simple_loss(f[:nb], g[:nb], ys[:nb], lx[:nb], ly[:nb], True, go, nthreads=cores)

    for _ in range(min(args.warmup, 1)):
        one()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        one()
    dt_s = time.perf_counter() - t0
    value = nb * args.steps / dt_s
    sample = f"every step = the first {nb} of {B} utterances on {cores} OpenMP threads"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": min(args.warmup, 1), "ms_per_step": 1e3 * dt_s / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": simple_workload_string(args.workload, 1)},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))
    return 0


def run_b200_simple(args):
    import torch
    import torch.distributed as dist

    from warp_ctct_b200 import _lib
    from warp_ctct_b200.sharded import plan_shards, shard_weights, sharded_ctct_simple_loss

    world, rank, local_rank, dev = setup_device(args)
    lib = _lib.lib()
    B, T, U1, V, lxr, lyr = SIMPLE_WORKLOADS[args.workload]
    lx_g, ly_g, ys_g = global_lengths(args.workload, world)
    plan = plan_shards(lx_g, ly_g, world)
    mine = np.array(plan[rank])
    lx, ly, ys = lx_g[mine], ly_g[mine], ys_g[mine]
    assert len(mine) == B
    G = B * world

    f_np, g_np = simple_inputs_host(args.workload, 2000 + rank)
    f_host = torch.from_numpy(f_np).pin_memory()
    g_host = torch.from_numpy(g_np).pin_memory()
    ys_h = torch.from_numpy(ys).pin_memory()
    lx_h = torch.from_numpy(lx).pin_memory()
    ly_h = torch.from_numpy(ly).pin_memory()
    f = f_host.to(dev).requires_grad_(True)
    g = g_host.to(dev).requires_grad_(True)
    ys_t, lx_t, ly_t = ys_h.to(dev), lx_h.to(dev), ly_h.to(dev)

    def step():
        f.grad = None
        g.grad = None
        loss = sharded_ctct_simple_loss(f, g, ys_t, lx_t, ly_t, global_batch=G, reduction="mean")
        loss.backward()
        return loss

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed_pass():
        """K steps between two events (barrier + synchronize on both sides), max over ranks."""
        barrier()
        ev0.record()
        t_host = time.perf_counter()
        for _ in range(args.steps):
            out = step()
        enqueue_us = 1e6 * (time.perf_counter() - t_host) / args.steps  # host time to enqueue one step
        ev1.record()
        barrier()
        t = torch.tensor([ev0.elapsed_time(ev1)], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()), enqueue_us, out

    # the timed region: nothing but the K steps
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    ms_total, host_us, loss = timed_pass()
    clocks = sampler.finish() if sampler else None

    # the same K steps once more with the library recording CUDA events around its kernels (the
    # event records between dependent launches cost a few microseconds per step, so this pass is
    # kept out of `value`): per-kernel durations for the roofline
    cap_n = 3 * args.steps + 3
    _lib.check(lib.ctct_b200_profile_enable(cap_n), "profile_enable")
    ms_profiled, _, _ = timed_pass()
    buf = np.zeros((cap_n, 4), np.float32)
    kinds = np.zeros((cap_n,), np.int32)
    n_rec = lib.ctct_b200_profile_read(buf.ctypes.data, kinds.ctypes.data, cap_n)
    lib.ctct_b200_profile_disable()
    rec = {k: buf[:n_rec][kinds[:n_rec] == k] for k in (3, 4, 5)}
    k_ms = {
        "exp_split": float(rec[3][:, 0].mean()), "logmm_tc": float(rec[3][:, 1].mean()),
        "logmm_exact_fixup": float(rec[3][:, 2].mean()),
        "compose": float(rec[4][:, 0].mean()), "lattice": float(rec[4][:, 1].mean()),
        "fill_grad": float(rec[4][:, 2].mean()),
        "den_backward_grad_f": float(rec[5][:, 0].mean()), "den_backward_grad_g": float(rec[5][:, 1].mean()),
        "label_patches": float(rec[5][:, 2].mean()),
    }
    value = G * args.steps / (ms_total * 1e-3)
    tc_peak, tc_kind = peaks("bf16_tflops", 1590.0)
    hbm_peak, hbm_kind = peaks()
    flops = 2.0 * B * T * U1 * V                       # one multiply-add per (t, u, v): the contraction itself
    tc_ach = flops / (k_ms["logmm_tc"] * 1e-3) / 1e12
    fused = U1 <= 128  # both gradients in one pass over the Ef planes (k_den_bwd_fused)
    if fused:
        # Ef planes (hi + lo) read, grad_f written, g read, grad_g written, Eg planes read
        gf_bytes = 4 * (2 * B * T * V) + 4 * (3 * B * U1 * V)
        gg_bytes = 0
        name = "k_den_bwd_fused (grad_f = Ef * (P Eg) and grad_g = Eg * (P^T Ef) in one pass: tcgen05 GEMMs) + k_den_weights"
    else:
        gf_bytes = 4 * (2 * B * T * V) + 4 * B * U1 * V    # f read, grad_f written, Eg planes (hi + lo) read
        gg_bytes = 4 * (2 * B * U1 * V) + 4 * B * T * V    # g read, grad_g written, Ef planes (hi + lo) read
        name = "k_logmm_bwd_tc (grad_f = Ef * (P Eg): tcgen05 GEMM with exp epilogue) + k_den_weights"
    gf_ach = gf_bytes / (k_ms["den_backward_grad_f"] * 1e-3) / 1e9
    # dominant launch of the step; it is bound by streaming the planes in and grad_f out, not by the tensor pipe
    roofline = {"kernel": name,
                "bound": "hbm", "achieved": gf_ach, "peak": hbm_peak, "unit": "GB/s", "frac": gf_ach / hbm_peak,
                "peak_source": f"of {hbm_kind}", "algorithmic_bytes": gf_bytes,
                "traffic": NCU_TRAFFIC_PER_LAUNCH.get(args.workload)}
    tensor = {"kernel": "k_logmm_tc (tcgen05 GEMM of the max-shifted exponentials, log/max epilogue)",
              "achieved": tc_ach, "peak": tc_peak, "unit": "TFLOP/s", "frac": tc_ach / tc_peak,
              "peak_source": f"of {tc_kind} (burst cuBLAS bf16)", "algorithmic_flops": flops, "issued_flops": 3 * flops,
              "note": "each product is issued as three bf16 MMAs (hi*hi, hi*lo, lo*hi) for float32-level accuracy; "
                      "at these shapes the kernel is bound by its operand planes (HBM/L2), not the tensor pipe"}
    plane_bytes = 2 * 2 * (B * T * V + B * U1 * V)      # bf16 hi+lo planes of both operands, read once
    split_bytes = 4 * (B * T * V + B * U1 * V) + plane_bytes
    kernels = {k: {"ms": v} for k, v in k_ms.items()}
    kernels["exp_split"].update({"GB/s": split_bytes / (k_ms["exp_split"] * 1e-3) / 1e9,
                                 "frac": split_bytes / (k_ms["exp_split"] * 1e-3) / 1e9 / hbm_peak})
    kernels["logmm_tc"].update({"TFLOP/s": tc_ach, "operand_GB/s": plane_bytes / (k_ms["logmm_tc"] * 1e-3) / 1e9,
                                "tensor_roofline": tensor})
    for key, nbytes in (("den_backward_grad_f", gf_bytes), ("den_backward_grad_g", gg_bytes)):
        if nbytes == 0:
            kernels[key]["note"] = "exact fall-back kernel only (a flag check); the fused kernel is in den_backward_grad_f"
            continue
        kernels[key].update({"GB/s": nbytes / (k_ms[key] * 1e-3) / 1e9, "frac": nbytes / (k_ms[key] * 1e-3) / 1e9 / hbm_peak,
                             "hbm_peak_source": f"of {hbm_kind}"})
    kernels["sum_ms"] = sum(k_ms.values())

    # ---- the same step captured once in a CUDA graph and replayed (single GPU; informational) ----
    graph_ms = None
    if world == 1:
        try:
            f_g, g_g = f.detach().requires_grad_(True), g.detach().requires_grad_(True)

            def graph_step():
                sharded_ctct_simple_loss(f_g, g_g, ys_t, lx_t, ly_t, global_batch=G, reduction="mean").backward()

            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(2):
                    f_g.grad = g_g.grad = None
                    graph_step()
            torch.cuda.current_stream().wait_stream(side)
            f_g.grad = g_g.grad = None
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                graph_step()
            for _ in range(3):
                graph.replay()
            torch.cuda.synchronize(dev)
            ev0.record()
            for _ in range(args.steps):
                graph.replay()
            ev1.record()
            torch.cuda.synchronize(dev)
            graph_ms = ev0.elapsed_time(ev1) / args.steps
            del graph, f_g, g_g
        except Exception as exc:  # capture is an extra: report why it did not happen
            graph_ms = f"not captured: {exc}"

    # ---- end to end: f and g copied from pinned host memory each step, loss read back ----
    e2e_steps = max(1, min(args.steps, args.e2e_steps))

    def e2e_step():
        a = f_host.to(dev, non_blocking=True).requires_grad_(True)
        b = g_host.to(dev, non_blocking=True).requires_grad_(True)
        y, p, q = ys_h.to(dev, non_blocking=True), lx_h.to(dev, non_blocking=True), ly_h.to(dev, non_blocking=True)
        out = sharded_ctct_simple_loss(a, b, y, p, q, global_batch=G, reduction="mean")
        out.backward()
        return float(out.item())

    for _ in range(2):
        e2e_step()
    barrier()
    ev0.record()
    for _ in range(e2e_steps):
        e2e_step()
    ev1.record()
    barrier()
    ms_e = torch.tensor([ev0.elapsed_time(ev1)], device=dev)
    if world > 1:
        dist.all_reduce(ms_e, op=dist.ReduceOp.MAX)
    h2d = 4 * (f_host.numel() + g_host.numel() + ys_h.numel() + lx_h.numel() + ly_h.numel())
    e2e = {"value": G * e2e_steps / (float(ms_e.item()) * 1e-3), "unit": UNIT, "h2d_bytes_per_step": int(h2d * world),
           "d2h_bytes_per_step": 4 * world, "steps": e2e_steps,
           "note": "f and g copied from pinned host memory every step; gradients stay on the device, the loss is read back"}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_total / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": simple_workload_string(args.workload, world),
                   "l2": f"inputs larger than L2: f {4 * B * T * V / 1e6:.0f} MB, g {4 * B * U1 * V / 1e6:.0f} MB, "
                         f"their gradients as much again, bf16 planes {plane_bytes / 1e6:.0f} MB (L2 is 126 MB)",
                   "shard_weights": shard_weights(lx_g, ly_g, plan)},
        "clocks": clocks, "e2e": e2e, "gpu_launches": (12 if U1 <= 128 else 13) * args.steps * world,
        "roofline": roofline, "kernels": kernels, "host_enqueue_us_per_step": host_us,
        "profiled_pass_ms_per_step": ms_profiled / args.steps,
    }
    if graph_ms is not None:
        line["cuda_graph_replay_ms_per_step"] = graph_ms
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        import oracle
        cores = oracle.max_threads()
        nb = min(B, 4)
        go = np.full((nb,), 1.0 / B, np.float32)
        t0 = time.perf_counter()
        costs_cpu, _, _ = oracle.simple_loss(f_np[:nb], g_np[:nb], ys[:nb], lx[:nb], ly[:nb], True, go, nthreads=cores)
        dt_s = time.perf_counter() - t0
        with torch.no_grad():
            from warp_ctct_b200 import ctct_simple_loss
            costs_gpu = ctct_simple_loss(f[:nb], g[:nb], ys_t[:nb], lx_t[:nb], ly_t[:nb], reduction="none").cpu().numpy()
        line["cpu_baseline"] = {"value": nb / dt_s, "unit": UNIT, "cores": cores, "kind": "port",
                                "sample": f"the first {nb} of {B} utterances, one pass, {cores} OpenMP threads; costs "
                                          f"agree with the GPU to {float(np.abs(costs_cpu - costs_gpu).max() / np.abs(costs_cpu).max()):.1e} rel"}
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS) + sorted(SIMPLE_WORKLOADS))
    ap.add_argument("--e2e-steps", type=int, default=20)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        if args.steps == 200 and "--steps" not in " ".join(sys.argv):
            args.steps, args.warmup = 10, 3
        return run_reference_simple(args) if args.workload in SIMPLE_WORKLOADS else run_reference(args)
    return run_b200_simple(args) if args.workload in SIMPLE_WORKLOADS else run_b200(args)


if __name__ == "__main__":
    sys.exit(main())
