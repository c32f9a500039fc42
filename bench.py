#!/usr/bin/env python
"""Benchmark of the CTC-Transducer loss hot path (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--passes R] [--impl b200|reference]
                    [--workload c2|c3|c5|c2_logits|c5_logits|c4|c4s|gather_probe] [--scaling weak|strong]

One "step" is one forward + backward of the loss over one batch of synthetic utterances per GPU.
Default workload ``c2``: float32 log-probs = log_softmax(1.5 * N(0,1)), B=32 per GPU, T=256, U+1=65,
V=512, frame lengths U[128,256], label lengths U[16,64] capped at frames/2.  ``*_logits`` workloads
feed raw scores to ``ctct_loss_from_logits`` (log-softmax fused into the kernels) and time the unfused
pipeline (torch.log_softmax + ctct_loss) beside it.  ``c4`` is ``ctct_simple_loss``.
With N > 1 (launched by torchrun, one rank per GPU) the global batch is split length-balanced over the
ranks; the only collective is the 4-byte all-reduce of the scalar loss.  ``--scaling weak`` (default)
keeps 32 utterances per GPU; ``--scaling strong`` keeps the global batch at 256 (32 per GPU at N=8).

Timing: W >= 3 warm-up steps plus more until 0.3 s have gone by (``warmup`` of the line is the number of
untimed steps actually run), then R passes (default 5) of exactly K steps, each pass bracketed by a
barrier + synchronize and timed with CUDA events, max over ranks; ``ms_per_step`` is the median pass,
the others are listed under ``passes``.  Inputs and outputs are far larger than L2.

Prints ONE JSON line (rank 0).  ``--impl reference`` times the CPU restatement of the reference's
algorithm (oracle/) on all host cores instead, on a bounded sample of the same workload.
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
STRONG_GLOBAL_BATCH = 256
METRIC = "utterances/sec fwd+bwd"
UNIT = "utt/s"


def base_name(name):
    for suffix in ("_packed", "_logits"):
        if name.endswith(suffix):
            name = name[:-len(suffix)]
    return name


def is_logits(name):
    return "_logits" in name


def is_packed(name):
    return name.endswith("_packed")


def per_gpu_batch(name, world, scaling):
    B = (SIMPLE_WORKLOADS[name][0] if name in SIMPLE_WORKLOADS else WORKLOADS[base_name(name)][0])
    if scaling == "strong":
        assert STRONG_GLOBAL_BATCH % world == 0
        return STRONG_GLOBAL_BATCH // world
    return B


def global_lengths(name, G, seed=2000):
    """Lengths and labels of the G utterances of the global batch (the same on every rank and arm)."""
    if name in SIMPLE_WORKLOADS:
        _, T, U1, V, lxr, lyr = SIMPLE_WORKLOADS[name]
        cap = False
    else:
        _, T, U1, V, dt, sigma, lxr, lyr, cap = WORKLOADS[base_name(name)]
    rng = np.random.default_rng(seed)
    lx = rng.integers(lxr[0], lxr[1] + 1, G).astype(np.int32)
    ly = rng.integers(lyr[0], lyr[1] + 1, G).astype(np.int32)
    if cap:
        ly = np.minimum(ly, lx // 2).astype(np.int32)
    ly = np.minimum(ly, lx).astype(np.int32)
    ys = rng.integers(1, V, (G, U1 - 1)).astype(np.int32)
    return lx, ly, ys


def make_config(name, world, scaling):
    """The `config` object of the JSON line: identical for the B200 arm and the reference arm."""
    from warp_ctct_b200.sharded import plan_shards, shard_weights
    B = per_gpu_batch(name, world, scaling)
    G = B * world
    lx, ly, _ = global_lengths(name, G)
    plan = plan_shards(lx, ly, world)
    if name in SIMPLE_WORKLOADS:
        _, T, U1, V, lxr, lyr = SIMPLE_WORKLOADS[name]
        text = (f"{name}: ctct_simple_loss f32 fwd+bwd (normalized), B={B}/GPU (global {G}), T={T}, U+1={U1}, "
                f"V={V}, f,g~N(0,1), lx~U{list(lxr)}, ly~U{list(lyr)}")
        l2 = (f"inputs larger than L2: f {4 * B * T * V / 1e6:.0f} MB, g {4 * B * U1 * V / 1e6:.0f} MB, their "
              f"gradients as much again, bf16 operand planes beside them (L2 is 126 MB)")
    else:
        _, T, U1, V, dt, sigma, lxr, lyr, cap = WORKLOADS[base_name(name)]
        esize = 4 if dt == "f32" else 2
        what = ("ctct_loss_from_logits: raw scores" if is_logits(name) else "ctct_loss: log_softmax of")
        if is_packed(name):
            what = "packed layout (valid rows only), " + what
        text = (f"{name}: {what} {sigma}*N(0,1), {dt} fwd+bwd, B={B}/GPU (global {G}), T={T}, U+1={U1}, V={V}, "
                f"lx~U{list(lxr)}, ly~U{list(lyr)}" + (" capped lx//2" if cap else ""))
        l2 = (f"inputs larger than L2: {B * T * U1 * V * esize / 1e9:.2f} GB joint tensor per GPU and an equally "
              f"large gradient written every step (L2 is 126 MB)")
    return {"workload": text, "scaling": scaling, "l2": l2, "shard_weights": shard_weights(lx, ly, plan)}


def peaks(key="hbm_gbs", fallback=6650.0):
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            return float(json.load(fh)[key]), "measured"
    except Exception:
        return fallback, "fallback"


def ncu_traffic(key):
    """DRAM bytes per launch of the dominant kernel from the committed ncu captures (profiles/ncu_traffic.json:
    which kernel, which capture, at which commit); None when no capture of this workload is on file."""
    try:
        with open(os.path.join(ROOT, "profiles", "ncu_traffic.json")) as fh:
            return json.load(fh)["workloads"][key]["dram_bytes_per_launch"]
    except Exception:
        return None


def host_cores():
    """Host threads this process may use (torchrun sets OMP_NUM_THREADS=1; the affinity mask is the truth)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    def __init__(self, device_index: int, period_s: float = 0.005):
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

def host_joint(name, B, seed=2000):
    """The synthetic joint tensor of one shard on the host (float32; 16-bit workloads rounded through the dtype)."""
    import torch
    _, T, U1, V, dt, sigma, _, _, _ = WORKLOADS[base_name(name)]
    gen = torch.Generator().manual_seed(seed)
    x = sigma * torch.randn((B, T, U1, V), generator=gen)
    if not is_logits(name):
        x = x.log_softmax(-1)
    if dt == "f16":
        x = x.half().float()
    return x


def cpu_step_standard(name, x, ys, lx, ly, go, cores):
    """One forward + backward of the reference's algorithm on the host: oracle/ for the loss; for a
    logits workload torch's CPU log_softmax in front of it and its backward behind, as a user of the
    reference would run them."""
    import torch

    import oracle
    if is_logits(name):
        lp = x.log_softmax(-1)
        costs, dense = oracle.ctct_loss(lp.numpy(), ys, lx, ly, go, nthreads=cores)
        d = torch.from_numpy(dense)
        grad = d - lp.exp() * d.sum(-1, keepdim=True)
        return costs, grad
    return oracle.ctct_loss(x.numpy(), ys, lx, ly, go, nthreads=cores)


def ref_py_baseline(name, x, ys, lx, ly, cores, budget_s=20.0):
    """The reference's own style of CPU path (per-cell Python loops over torch scalars, as its
    ref_ctct.py does; restated in oracle/ref_py.py), one process per core on the first utterances of
    the batch, extrapolated to utterances/s on all cores."""
    try:
        from oracle import ref_py
    except Exception as exc:  # pragma: no cover
        return {"unavailable": f"oracle.ref_py not importable: {exc}"}
    n = int(min(len(lx), cores, 8))
    t0 = time.perf_counter()
    per_utt = ref_py.time_utterances(x[:n].numpy(), ys[:n], lx[:n], ly[:n], processes=n, budget_s=budget_s)
    wall = time.perf_counter() - t0
    if not per_utt:
        return {"unavailable": "no utterance finished within the time budget"}
    mean_s = float(np.mean(per_utt))
    return {"value": cores / mean_s, "unit": UNIT, "cores": cores, "kind": "port-python",
            "sample": f"first {len(per_utt)} utterances, one single-threaded process each (forward and backward "
                      f"variables + occupancy gradient in per-cell Python loops), {mean_s:.2f} s per utterance per "
                      f"core, extrapolated to {cores} cores; wall {wall:.1f} s"}


def run_reference(args):
    """CPU arm: the C restatement of the reference's algorithm (oracle/) on all host threads; every
    step is one shard (the per-GPU batch) of the workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    import torch
    world = max(1, args.gpus)
    cores = host_cores()
    torch.set_num_threads(cores)
    name = args.workload
    _, T, U1, V, dt, sigma, lxr, lyr, cap = WORKLOADS[base_name(name)]
    B = per_gpu_batch(name, world, args.scaling)
    G = B * world
    lx_g, ly_g, ys_g = global_lengths(name, G)
    from warp_ctct_b200.sharded import plan_shards
    mine = np.array(plan_shards(lx_g, ly_g, world)[0])
    nb = min(B, 32)                       # bounded sample: at most 32 utterances per step
    mine = mine[:nb]
    lx, ly, ys = lx_g[mine], ly_g[mine], ys_g[mine]
    x = host_joint(name, nb)
    go = np.full((nb,), 1.0 / G, np.float32)
    for _ in range(args.warmup):
        cpu_step_standard(name, x, ys, lx, ly, go, cores)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_step_standard(name, x, ys, lx, ly, go, cores)
    dt_s = time.perf_counter() - t0
    value = nb * args.steps / dt_s
    sample = (f"every step = {nb} utterances (rank 0's shard of the global batch of {G}) on {cores} host threads "
              f"(OpenMP C port of the reference's algorithm" + ("; torch CPU log_softmax around it" if is_logits(name) else "") + ")")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt_s / args.steps,
        "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": dt, "data": "synthetic",
        "config": make_config(name, world, args.scaling),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
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


class Timer:
    """K steps between two CUDA events, barrier + synchronize on both sides, max over ranks."""

    def __init__(self, world, dev):
        import torch
        self.torch, self.world, self.dev = torch, world, dev
        self.ev0, self.ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def barrier(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        self.torch.cuda.synchronize(self.dev)

    def timed(self, fn, n):
        """Returns (ms for n calls, host microseconds to enqueue one call, last result)."""
        self.barrier()
        self.ev0.record()
        t_host = time.perf_counter()
        out = None
        for _ in range(n):
            out = fn()
        enqueue_us = 1e6 * (time.perf_counter() - t_host) / max(n, 1)
        self.ev1.record()
        self.barrier()
        t = self.torch.tensor([self.ev0.elapsed_time(self.ev1), enqueue_us], device=self.dev)
        if self.world > 1:
            import torch.distributed as dist
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        # both figures are the maximum over ranks: the slowest GPU and the slowest host thread set the pace
        return float(t[0].item()), float(t[1].item()), out

    def passes(self, fn, steps, n_passes):
        """R passes of K steps: per-pass ms per step, host enqueue time, last result."""
        per, host, out = [], [], None
        for _ in range(n_passes):
            ms, us, out = self.timed(fn, steps)
            per.append(ms / steps)
            host.append(us)
        return per, statistics.median(host), out


def settle(step, warmup, world, seconds=0.3):
    """The W warm-up steps, then more of them until `seconds` of wall time have gone by: with several ranks per
    box the first tenth of a second of a run is slower than the rest (the first two passes of 40 ms each took 0.25
    instead of 0.21 ms per step at 8 GPUs), and the timed passes should not start inside it.  The ranks go on in
    rounds of 50 steps and agree after each round whether to stop, so that all run the same number of steps.
    Returns the number of untimed steps."""
    import torch
    for _ in range(warmup):
        step()
    extra, t0 = 0, time.perf_counter()
    while True:
        for _ in range(50):
            step()
        extra += 50
        stop = time.perf_counter() - t0 >= seconds
        if world > 1:
            import torch.distributed as dist
            flag = torch.tensor([1 if stop else 0], dtype=torch.int32, device="cuda")
            dist.all_reduce(flag, op=dist.ReduceOp.MAX)
            stop = bool(flag.item())
        if stop:
            return warmup + extra


def pass_stats(per):
    med = statistics.median(per)
    return {"n": len(per), "ms_per_step": [round(p, 6) for p in per], "median": med, "min": min(per), "max": max(per),
            "spread": (max(per) - min(per)) / med if med > 0 else None}


def read_profile(lib, cap_n):
    buf = np.zeros((cap_n, 4), np.float32)
    kinds = np.zeros((cap_n,), np.int32)
    n_rec = lib.ctct_b200_profile_read(buf.ctypes.data, kinds.ctypes.data, cap_n)
    lib.ctct_b200_profile_disable()
    return buf[:max(n_rec, 0)], kinds[:max(n_rec, 0)]


def standard_inputs(name, B, rank, dev):
    import torch
    _, T, U1, V, dt, sigma, _, _, _ = WORKLOADS[base_name(name)]
    tdt = {"f32": torch.float32, "f16": torch.float16}[dt]
    gen = torch.Generator(device=dev).manual_seed(2000 + rank)
    x = torch.empty((B, T, U1, V), dtype=tdt, device=dev)
    for n0 in range(0, B, 16):     # a few utterances at a time: the float32 intermediate stays small
        n1 = min(B, n0 + 16)
        y = sigma * torch.randn((n1 - n0, T, U1, V), device=dev, generator=gen)
        x[n0:n1] = (y if is_logits(name) else y.log_softmax(-1)).to(tdt)
    return x


def measure_standard(args, name, world, rank, local_rank, dev, timer, primary=True):
    """Times one standard-loss workload (c2 / c3 / c5, plain or from logits).  Returns the dict of its figures."""
    import torch
    import torch.distributed as dist

    import warp_ctct_b200 as W
    from warp_ctct_b200 import _lib
    from warp_ctct_b200.sharded import plan_shards, sharded_ctct_loss

    lib = _lib.lib()
    _, T, U1, V, dt, sigma, lxr, lyr, cap = WORKLOADS[base_name(name)]
    logits = is_logits(name)
    packed = is_packed(name)
    esize = {"f32": 4, "f16": 2}[dt]
    B = per_gpu_batch(name, world, args.scaling)
    G = B * world
    lx_g, ly_g, ys_g = global_lengths(name, G)
    plan = plan_shards(lx_g, ly_g, world)
    mine = np.array(plan[rank])
    lx, ly, ys = lx_g[mine], ly_g[mine], ys_g[mine]
    assert len(mine) == B
    lp = standard_inputs(name, B, rank, dev)
    ys_t, lx_t, ly_t = (torch.from_numpy(a).to(dev) for a in (ys, lx, ly))
    if packed:
        lp = W.pack_joint(lp, lx_t, ly_t).contiguous()
        torch.cuda.empty_cache()
    lp.requires_grad_(True)
    steps = args.steps if primary else max(10, min(args.steps, 100))
    n_passes = args.passes if primary else min(args.passes, 3)

    def loss_of(x, y, a, b):
        if packed:
            loss_p = W.ctct_loss_packed(x, y, a, b, reduction="mean", max_frames=T, from_logits=logits, global_batch=G)
            if world > 1:
                from warp_ctct_b200.sharded import all_reduce_sum
                loss_p = all_reduce_sum(loss_p)
            return loss_p
        return sharded_ctct_loss(x, y, a, b, global_batch=G, reduction="mean", from_logits=logits)

    def step():
        lp.grad = None
        loss = loss_of(lp, ys_t, lx_t, ly_t)
        loss.backward()
        return loss

    warm = settle(step, max(args.warmup, 3), world)
    timer.barrier()

    sampler = ClockSampler(local_rank) if (rank == 0 and primary) else None
    if sampler:
        sampler.start()
    per, host_us, loss = timer.passes(step, steps, n_passes)
    clocks = sampler.finish() if sampler else None
    ms_step = statistics.median(per)
    loss_value = float(loss.item())
    res = {"value": G / (ms_step * 1e-3), "ms_per_step": ms_step, "passes": pass_stats(per), "steps": steps, "warmup_steps": warm,
           "global_batch": G, "clocks": clocks, "host_enqueue_us_per_step": host_us, "loss": loss_value}

    # the same K steps once more with the library recording CUDA events around its kernels (the event
    # records between dependent launches cost a few microseconds per step, so this pass is kept out of
    # `value`): per-kernel durations for the roofline
    cap_n = 3 * steps + 3
    _lib.check(lib.ctct_b200_profile_enable(cap_n), "profile_enable")
    ms_profiled, _, _ = timer.timed(step, steps)
    buf, kinds = read_profile(lib, cap_n)
    fwd = buf[kinds == (6 if logits else 0)]
    bwd = buf[kinds == (7 if logits else 1)]
    res["profiled_pass_ms_per_step"] = ms_profiled / steps
    peak, peak_kind = peaks()
    rows_valid = int((lx.astype(np.int64) * (ly + 1)).sum())
    valid_bytes = rows_valid * V * esize
    full_bytes = valid_bytes if packed else B * T * U1 * V * esize   # a packed tensor has no padding rows
    precleared = (not logits) and (packed or (bool(W.PREZERO) and full_bytes >= W.PREZERO_MIN_BYTES))
    kernels = {}
    if logits:
        k_ms = {"lse_gather": float(fwd[:, 0].mean()), "lattice": float(fwd[:, 1].mean()),
                "fill_grad": float(fwd[:, 2].mean()), "logits_grad": float(bwd[:, 0].mean())}
        # with the gradient buffer allocated in the forward pass the lattice launch zeroes the padding rows
        # and the backward kernel reads and writes valid rows only; else it also writes the padding
        pad_cleared = (not packed) and bool(W.PREZERO) and full_bytes >= W.PREZERO_MIN_BYTES and (V * esize) % 16 == 0
        bwd_bytes = 2 * valid_bytes if pad_cleared else valid_bytes + full_bytes
        ach = bwd_bytes / (k_ms["logits_grad"] * 1e-3) / 1e9
        fwd_ach = valid_bytes / (k_ms["lse_gather"] * 1e-3) / 1e9
        roofline = {"kernel": "k_logits_grad (d loss / d logits = G - softmax * sum G: valid rows read once and written once"
                              + ("; padding rows were zeroed under the lattice)" if pad_cleared else ", padding rows written as zeros)"),
                    "bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                    "peak_source": f"of {peak_kind}", "algorithmic_bytes": bwd_bytes, "traffic": ncu_traffic(name)}
        kernels["lse_gather"] = {"ms": k_ms["lse_gather"], "algorithmic_bytes": valid_bytes, "GB/s": fwd_ach,
                                 "frac": fwd_ach / peak, "note": "valid rows read once: row log-sum-exp + the three picks"}
        if pad_cleared:
            pad_ach = (full_bytes - valid_bytes) / (k_ms["lattice"] * 1e-3) / 1e9
            kernels["lattice_and_pad_clear"] = {"ms": k_ms["lattice"], "algorithmic_bytes": full_bytes - valid_bytes,
                                                "GB/s": pad_ach, "frac": pad_ach / peak,
                                                "note": "one launch: 2 lattice CTAs per utterance + one block per (n,t) slab "
                                                        "that zeroes the slab's padding rows of the gradient"}
        else:
            kernels["lattice"] = {"ms": k_ms["lattice"], "ns_per_row": 1e6 * k_ms["lattice"] / max(int(lx.max()), 1)}
        kernels["fill_grad"] = {"ms": k_ms["fill_grad"]}
        kernels["logits_grad"] = {"ms": k_ms["logits_grad"], "GB/s": ach, "frac": ach / peak}
        kernels["valid_fraction_of_rows"] = rows_valid / (B * T * U1)
    else:
        k_ms = {"gather": float(fwd[:, 0].mean()), "lattice": float(fwd[:, 1].mean()), "fill_grad": float(fwd[:, 2].mean())}
        k_ms["dense_patch" if precleared else "dense_grad"] = float(bwd[:, 0].mean())
        dense_key = "lattice" if precleared else "dense_grad"
        dense_bytes = full_bytes if precleared else full_bytes + rows_valid * 16
        gather_bytes = rows_valid * 3 * 32 + B * T * U1 * 16    # one 32-byte sector per picked element + records out
        ach = dense_bytes / (k_ms[dense_key] * 1e-3) / 1e9
        roofline = {"kernel": ("k_lattice, clearing role (dense gradient streamer; shares the launch with the lattice CTAs)"
                               if precleared else "k_dense_grad (dense gradient streamer)"),
                    "bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                    "peak_source": f"of {peak_kind}", "algorithmic_bytes": dense_bytes, "traffic": ncu_traffic(name)}
        g_ach = gather_bytes / (k_ms["gather"] * 1e-3) / 1e9
        kernels["gather"] = {"ms": k_ms["gather"], "sector_bytes": gather_bytes, "GB/s": g_ach, "frac": g_ach / peak,
                             "isolated_reads_per_s": rows_valid * 3 / (k_ms["gather"] * 1e-3)}
        kernels["fill_grad"] = {"ms": k_ms["fill_grad"]}
        if precleared:
            kernels["lattice_and_clear"] = {"ms": k_ms["lattice"], "GB/s": ach, "frac": ach / peak,
                                            "note": "one launch: 2 lattice CTAs per utterance + blocks that zero the gradient"}
            kernels["dense_patch"] = {"ms": k_ms["dense_patch"]}
        else:
            kernels["lattice"] = {"ms": k_ms["lattice"], "ns_per_row": 1e6 * k_ms["lattice"] / max(int(lx.max()), 1)}
            kernels["dense_grad"] = {"ms": k_ms["dense_grad"], "GB/s": ach, "frac": ach / peak}
    kernels["sum_ms"] = sum(k_ms.values())
    # whole-step floor: the bytes the step cannot avoid at the measured peak
    floor_bytes = (2 * valid_bytes + full_bytes) if logits else full_bytes
    res["step_floor"] = {"bytes": floor_bytes, "ms_at_peak": floor_bytes / (peak * 1e9) * 1e3,
                         "frac": floor_bytes / (peak * 1e9) * 1e3 / ms_step,
                         "note": ("valid rows read twice + every row written once" if logits else
                                  "the dense gradient written once") + f", at the {peak_kind} HBM peak"}
    res["roofline"], res["kernels"] = roofline, kernels

    if primary and precleared and not packed:
        # the lattice recursion by itself: a few steps with the clearing moved out of its launch
        W.PREZERO = False
        try:
            n_alone = 10
            _lib.check(lib.ctct_b200_profile_enable(3 * n_alone), "profile_enable")
            for _ in range(n_alone):
                step()
            torch.cuda.synchronize(dev)
            buf2, kinds2 = read_profile(lib, 3 * n_alone)
            alone = buf2[kinds2 == 0][:, 1]
            kernels["lattice_alone"] = {"ms": float(alone.mean()), "ns_per_row": 1e6 * float(alone.mean()) / max(int(lx.max()), 1),
                                        "note": "alpha and beta CTAs of all utterances run concurrently; rows = frames of "
                                                "the longest utterance; measured with the clearing blocks taken out"}
        finally:
            W.PREZERO = True

    if logits:
        # the unfused pipeline on the same logits: torch.log_softmax, this library's ctct_loss, autograd back through both
        def unfused():
            lp.grad = None
            if packed:
                loss_u = W.ctct_loss_packed(lp.log_softmax(-1), ys_t, lx_t, ly_t, reduction="mean", max_frames=T, global_batch=G)
            else:
                loss_u = sharded_ctct_loss(lp.log_softmax(-1), ys_t, lx_t, ly_t, global_batch=G, reduction="mean")
            loss_u.backward()
            return loss_u

        for _ in range(3):
            unfused()
        per_u, _, loss_u = timer.passes(unfused, max(5, steps // 4), min(n_passes, 3))
        ms_u = statistics.median(per_u)
        res["unfused"] = {"ms_per_step": ms_u, "value": G / (ms_u * 1e-3), "speedup_of_fused": ms_u / ms_step,
                          "loss_rel_diff": abs(float(loss_u.item()) - loss_value) / abs(loss_value),
                          "what": "torch.log_softmax + warp_ctct_b200.ctct_loss + autograd through both"}
        lp.grad = None

    if not primary:
        del lp
        torch.cuda.empty_cache()
        return res

    # ---- the same step captured once in a CUDA graph and replayed (single GPU; informational) ----
    if world == 1:
        try:
            lp_g = lp.detach().requires_grad_(True)   # a fresh leaf: its gradient accumulator belongs to the capturing stream

            def graph_step():
                loss_of(lp_g, ys_t, lx_t, ly_t).backward()

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
            ms_g, _, _ = timer.timed(graph.replay, steps)
            res["cuda_graph_replay_ms_per_step"] = ms_g / steps
            del graph, lp_g
        except Exception as exc:  # capture is an extra: report why it did not happen
            res["cuda_graph_replay_ms_per_step"] = f"not captured: {exc}"
        lp.grad = None

    if args.no_e2e:
        res["e2e"] = None
        res["_host"] = (lp.detach().cpu(), ys, lx, ly)
        return res

    # ---- end to end through the public API, inputs in pinned host memory ----
    e2e_steps = max(1, min(args.steps, args.e2e_steps))
    tdt = lp.dtype
    lp_host = torch.empty(tuple(lp.shape), dtype=tdt, pin_memory=True)
    lp_host.copy_(lp.detach())
    grad_host = torch.empty(tuple(lp.shape), dtype=tdt, pin_memory=True)
    ys_h, lx_h, ly_h = ys_t.cpu().pin_memory(), lx_t.cpu().pin_memory(), ly_t.cpu().pin_memory()
    del lp
    torch.cuda.empty_cache()
    small = 4 * (ys_h.numel() + lx_h.numel() + ly_h.numel())

    def copy_in():
        x = lp_host.to(dev, non_blocking=True).requires_grad_(True)
        return x, ys_h.to(dev, non_blocking=True), lx_h.to(dev, non_blocking=True), ly_h.to(dev, non_blocking=True)

    def e2e_full_copy():
        # the whole joint tensor crosses PCIe, then the usual autograd path; the loss is read back
        x, y, a, b = copy_in()
        loss = loss_of(x, y, a, b)
        loss.backward()
        return float(loss.item())

    def e2e_full_copy_grad_back():
        # ... and the dense gradient is copied back into pinned host memory as well
        x, y, a, b = copy_in()
        loss = loss_of(x, y, a, b)
        loss.backward()
        grad_host.copy_(x.grad, non_blocking=True)
        return float(loss.item())

    def e2e_in_place():
        # the joint tensor stays in pinned host memory: the gather kernel reads the three log-probs it
        # needs per row in place over PCIe; labels and lengths are copied; the loss is read back
        loss, grad = W.ctct_loss_and_grad(lp_host, ys_h, lx_h, ly_h, reduction="mean", device=dev, global_batch=G)
        if world > 1:
            dist.all_reduce(loss)
        return float(loss.item())

    def timed_e2e(fn):
        for _ in range(2):
            fn()
        ms, _, _ = timer.timed(fn, e2e_steps)
        return G * e2e_steps / (ms * 1e-3)

    full_h2d = int((lp_host.numel() * esize + small) * world)
    variants = {
        "full_copy": {"value": timed_e2e(e2e_full_copy), "unit": UNIT, "h2d_bytes_per_step": full_h2d,
                      "d2h_bytes_per_step": 4 * world,
                      "note": "whole joint tensor copied host to device every step, autograd path, gradient stays on the "
                              "device, loss read back"},
        "full_copy_grad_back": {"value": timed_e2e(e2e_full_copy_grad_back), "unit": UNIT, "h2d_bytes_per_step": full_h2d,
                                "d2h_bytes_per_step": int((lp_host.numel() * esize + 4) * world),
                                "note": "as full_copy, and the dense gradient copied back to pinned host memory"},
    }
    if not logits and not packed:
        variants["in_place"] = {
            "value": timed_e2e(e2e_in_place), "unit": UNIT,
            "h2d_bytes_per_step": int((rows_valid * 3 * 32 + small) * world), "d2h_bytes_per_step": 4 * world,
            "note": "ctct_loss_and_grad on the joint tensor left in pinned host memory: the gather kernel reads the 3 "
                    "log-probs per valid row in place over PCIe (one 32-byte sector each), labels and lengths are "
                    "copied, the dense gradient stays on the device, the loss scalar is read back"}
    head = "full_copy" if (logits or packed) else "in_place"
    res["e2e"] = {"value": variants[head]["value"], "unit": UNIT,
                  "h2d_bytes_per_step": variants[head]["h2d_bytes_per_step"],
                  "d2h_bytes_per_step": variants[head]["d2h_bytes_per_step"], "steps": e2e_steps, "variant": head,
                  "note": variants[head]["note"], "variants": variants}
    res["_host"] = (lp_host, ys, lx, ly)
    return res


def run_b200(args):
    import torch
    import torch.distributed as dist

    world, rank, local_rank, dev = setup_device(args)
    timer = Timer(world, dev)
    name = args.workload
    _, T, U1, V, dt, sigma, lxr, lyr, cap = WORKLOADS[base_name(name)]
    res = measure_standard(args, name, world, rank, local_rank, dev, timer, primary=True)
    lp_host, ys, lx, ly = res.pop("_host")
    B = per_gpu_batch(name, world, args.scaling)
    G = B * world
    launches_per_step = 4
    line = {
        "metric": METRIC, "value": res["value"], "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": res["warmup_steps"], "ms_per_step": res["ms_per_step"], "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None, "dtype": dt, "data": "synthetic",
        "config": make_config(name, world, args.scaling),
        "clocks": res["clocks"], "e2e": res["e2e"], "gpu_launches": launches_per_step * args.steps * args.passes * world,
        "gpu_launches_note": f"{launches_per_step} kernels of this library per step x {args.steps} steps x {args.passes} "
                             f"timed passes x {world} GPUs",
        "passes": res["passes"], "roofline": res["roofline"], "kernels": res["kernels"], "step_floor": res["step_floor"],
        "host_enqueue_us_per_step": res["host_enqueue_us_per_step"],
        "profiled_pass_ms_per_step": res["profiled_pass_ms_per_step"],
    }
    for key in ("cuda_graph_replay_ms_per_step", "unfused"):
        if key in res:
            line[key] = res[key]

    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cores = host_cores()
        torch.set_num_threads(cores)
        go = np.full((B,), 1.0 / G, np.float32)
        nb = min(B, 32)
        if is_packed(name):   # the CPU code takes the padded form (it skips padding rows itself)
            from warp_ctct_b200.packed import unpack_joint
            lp_host = unpack_joint(lp_host.float(), torch.from_numpy(lx), torch.from_numpy(ly), T, U1)
        xs, yb, lxb, lyb, gob = lp_host[:nb].float(), ys[:nb], lx[:nb], ly[:nb], go[:nb]
        cpu_step_standard(name, xs, yb, lxb, lyb, gob, cores)
        reps, t0 = 0, time.perf_counter()
        while reps < 3 or (time.perf_counter() - t0 < 3.0 and reps < 500):   # a bounded sample: about 3 s of all cores
            costs_cpu, _ = cpu_step_standard(name, xs, yb, lxb, lyb, gob, cores)
            reps += 1
        dt_s = (time.perf_counter() - t0) / reps
        sample = (f"{nb} utterances of the batch, mean of {reps} passes, {cores} host threads (OpenMP C port of the "
                  f"reference's algorithm" + ("; torch CPU log_softmax around it" if is_logits(name) else "") + ")")
        if nb == B:
            sample += f"; loss agrees with the GPU to {abs(float(costs_cpu.mean()) - res['loss']) / abs(res['loss']):.1e} rel"
        line["cpu_baseline"] = {"value": nb / dt_s, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample,
                                "ref_py": ref_py_baseline(name, xs.log_softmax(-1) if is_logits(name) else xs,
                                                          yb, lxb, lyb, cores)}
    del lp_host

    # the sharded configuration the scaling target is quoted on (c5: B=256 at 8 GPUs), in the same line
    if name == "c2" and not args.no_extra:
        extra = measure_standard(args, "c5", world, rank, local_rank, dev, timer, primary=False)
        line["workloads"] = {"c5": {"value": extra["value"], "unit": UNIT, "ms_per_step": extra["ms_per_step"],
                                    "global_batch": extra["global_batch"], "passes": extra["passes"],
                                    "roofline": extra["roofline"], "config": make_config("c5", world, args.scaling)}}
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        from warp_ctct_b200.sharded import close_scalar_comms
        dist.barrier()
        close_scalar_comms()
        dist.destroy_process_group()
    return 0


# --------------------------------------------------------------------------------------- gather probe

def run_gather_probe(args):
    """How fast can isolated 4-byte reads (one per 2 KB vocabulary row, each its own DRAM sector) be issued?
    The gather of workload c2, timed alone with CUDA events, for several numbers of loads in flight
    per thread and resident blocks per SM."""
    import torch

    from warp_ctct_b200 import _lib
    args.gpus = 1
    world, rank, local_rank, dev = setup_device(args)
    lib = _lib.lib()
    B, T, U1, V, dt, sigma, lxr, lyr, cap = WORKLOADS["c2"]
    lx, ly, ys = global_lengths("c2", B)
    lp = standard_inputs("c2", B, 0, dev)
    ys_t, lx_t, ly_t = (torch.from_numpy(a).to(dev) for a in (ys, lx, ly))
    out = torch.empty((B, T, U1, 4), dtype=torch.float32, device=dev)
    flush = torch.empty((256 << 20,), dtype=torch.uint8, device=dev)
    rows_valid = int((lx.astype(np.int64) * (ly + 1)).sum())
    reads = rows_valid * 3
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    st = _lib.stream_ptr(dev)
    results = []
    for per in (1, 2, 4, 8, 16):
        for bps in (2, 4, 8, 16, 0):     # 0 = one thread per element group, as many blocks as it takes
            times = []
            for it in range(max(args.steps, 5) + 3):
                flush.zero_()             # the joint tensor (1.09 GB) does not fit L2 anyway; this also evicts the records
                ev0.record()
                rc = lib.ctct_b200_gather_probe(lp.data_ptr(), ys_t.data_ptr(), lx_t.data_ptr(), ly_t.data_ptr(), B, T, U1, V,
                                                per, bps, out.data_ptr(), st)
                ev1.record()
                _lib.check(rc, "gather_probe")
                torch.cuda.synchronize(dev)
                if it >= 3:
                    times.append(ev0.elapsed_time(ev1) * 1e3)
            us = statistics.median(times)
            results.append({"loads_per_thread": per, "blocks_per_sm": bps if bps else "unbounded", "us": us,
                            "isolated_reads_per_s": reads / (us * 1e-6), "sector_GB/s": reads * 32 / (us * 1e-6) / 1e9})
    best = min(results, key=lambda r: r["us"])
    peak, peak_kind = peaks()
    line = {"metric": "isolated 4-byte DRAM reads per second (gather of workload c2, kernel alone)",
            "value": best["isolated_reads_per_s"], "unit": "reads/s", "n_gpus": 1, "steps": max(args.steps, 5), "warmup": 3,
            "ms_per_step": best["us"] * 1e-3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"gather_probe: k_gather3 variants on the c2 joint tensor ({reads} reads, one 32-byte "
                                   f"sector each; L2 flushed between launches)"},
            "best": best, "variants": results,
            "roofline": {"bound": "hbm", "achieved": best["sector_GB/s"], "peak": peak, "unit": "GB/s",
                         "frac": best["sector_GB/s"] / peak, "peak_source": f"of {peak_kind}", "traffic": None,
                         "note": "sector bytes (32 per read) over the best variant's time"}}
    print(json.dumps(line))
    return 0


# --------------------------------------------------------------------------------------- ctct_simple_loss (c4)

def simple_inputs_host(name, B, seed=2000):
    _, T, U1, V, lxr, lyr = SIMPLE_WORKLOADS[name]
    rng = np.random.default_rng(seed)
    f = rng.standard_normal((B, T, V), dtype=np.float32)
    g = rng.standard_normal((B, U1, V), dtype=np.float32)
    return f, g


def run_reference_simple(args):
    """CPU arm for the log-add-joiner loss: the C restatement on all host threads, on a bounded
    sample of the batch (the first utterances) so that a run ends within minutes."""
    if int(os.environ.get("RANK", "0")) != 0:
        return 0
    import oracle
    name = args.workload
    world = max(1, args.gpus)
    _, T, U1, V, lxr, lyr = SIMPLE_WORKLOADS[name]
    B = per_gpu_batch(name, world, args.scaling)
    G = B * world
    lx_g, ly_g, ys_g = global_lengths(name, G)
    from warp_ctct_b200.sharded import plan_shards
    nb = min(B, 4)
    mine = np.array(plan_shards(lx_g, ly_g, world)[0])[:nb]
    lx, ly, ys = lx_g[mine], ly_g[mine], ys_g[mine]
    f, g = simple_inputs_host(name, nb)
    cores = host_cores()
    go = np.full((nb,), 1.0 / G, np.float32)

    def one():
        return oracle.simple_loss(f, g, ys, lx, ly, True, go, nthreads=cores)

    for _ in range(min(args.warmup, 1)):
        one()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        one()
    dt_s = time.perf_counter() - t0
    value = nb * args.steps / dt_s
    sample = f"every step = {nb} utterances of rank 0's shard on {cores} host threads (OpenMP C port)"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": min(args.warmup, 1), "ms_per_step": 1e3 * dt_s / args.steps,
        "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": make_config(name, world, args.scaling),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))
    return 0


def run_b200_simple(args):
    import torch
    import torch.distributed as dist

    from warp_ctct_b200 import _lib
    from warp_ctct_b200.sharded import plan_shards, sharded_ctct_simple_loss

    world, rank, local_rank, dev = setup_device(args)
    timer = Timer(world, dev)
    lib = _lib.lib()
    name = args.workload
    _, T, U1, V, lxr, lyr = SIMPLE_WORKLOADS[name]
    B = per_gpu_batch(name, world, args.scaling)
    G = B * world
    lx_g, ly_g, ys_g = global_lengths(name, G)
    plan = plan_shards(lx_g, ly_g, world)
    mine = np.array(plan[rank])
    lx, ly, ys = lx_g[mine], ly_g[mine], ys_g[mine]
    assert len(mine) == B

    f_np, g_np = simple_inputs_host(name, B, 2000 + rank)
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

    warm = settle(step, max(args.warmup, 3), world)
    timer.barrier()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    per, host_us, loss = timer.passes(step, args.steps, args.passes)
    clocks = sampler.finish() if sampler else None
    ms_step = statistics.median(per)

    cap_n = 3 * args.steps + 3
    _lib.check(lib.ctct_b200_profile_enable(cap_n), "profile_enable")
    ms_profiled, _, _ = timer.timed(step, args.steps)
    buf, kinds = read_profile(lib, cap_n)
    rec = {k: buf[kinds == k] for k in (3, 4, 5)}
    k_ms = {
        "exp_split": float(rec[3][:, 0].mean()), "logmm_tc": float(rec[3][:, 1].mean()),
        "logmm_exact_fixup": float(rec[3][:, 2].mean()),
        "compose": float(rec[4][:, 0].mean()), "lattice": float(rec[4][:, 1].mean()),
        "fill_grad": float(rec[4][:, 2].mean()),
        "den_backward_grad_f": float(rec[5][:, 0].mean()), "den_backward_grad_g": float(rec[5][:, 1].mean()),
        "label_patches": float(rec[5][:, 2].mean()),
    }
    value = G / (ms_step * 1e-3)
    tc_peak, tc_kind = peaks("bf16_tflops", 1590.0)
    hbm_peak, hbm_kind = peaks()
    flops = 2.0 * B * T * U1 * V                       # one multiply-add per (t, u, v): the contraction itself
    tc_ach = flops / (k_ms["logmm_tc"] * 1e-3) / 1e12
    fused = U1 <= 128  # both gradients in one pass over the Ef planes (k_den_bwd_fused)
    if fused:
        # Ef planes (hi + lo) read, grad_f written, g read, grad_g written, Eg planes read
        gf_bytes = 4 * (2 * B * T * V) + 4 * (3 * B * U1 * V)
        gg_bytes = 0
        kname = "k_den_bwd_fused (grad_f = Ef * (P Eg) and grad_g = Eg * (P^T Ef) in one pass: tcgen05 GEMMs) + k_den_weights"
    else:
        gf_bytes = 4 * (2 * B * T * V) + 4 * B * U1 * V    # f read, grad_f written, Eg planes (hi + lo) read
        gg_bytes = 4 * (2 * B * U1 * V) + 4 * B * T * V    # g read, grad_g written, Ef planes (hi + lo) read
        kname = "k_logmm_bwd_tc (grad_f = Ef * (P Eg): tcgen05 GEMM with exp epilogue) + k_den_weights"
    gf_ach = gf_bytes / (k_ms["den_backward_grad_f"] * 1e-3) / 1e9
    roofline = {"kernel": kname,
                "bound": "hbm", "achieved": gf_ach, "peak": hbm_peak, "unit": "GB/s", "frac": gf_ach / hbm_peak,
                "peak_source": f"of {hbm_kind}", "algorithmic_bytes": gf_bytes, "traffic": ncu_traffic(name)}
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
    floor_bytes = 4 * 2 * (B * T * V + B * U1 * V)      # f, g read; grad_f, grad_g written
    step_floor = {"bytes": floor_bytes, "ms_at_peak": floor_bytes / (hbm_peak * 1e9) * 1e3,
                  "frac": floor_bytes / (hbm_peak * 1e9) * 1e3 / ms_step,
                  "note": f"f and g read once, their gradients written once, at the {hbm_kind} HBM peak"}

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
            ms_g, _, _ = timer.timed(graph.replay, args.steps)
            graph_ms = ms_g / args.steps
            del graph, f_g, g_g
        except Exception as exc:  # capture is an extra: report why it did not happen
            graph_ms = f"not captured: {exc}"

    # ---- end to end: f and g copied from pinned host memory each step, loss read back ----
    e2e_steps = max(1, min(args.steps, args.e2e_steps))
    gf_host = torch.empty_like(f_host).pin_memory()
    gg_host = torch.empty_like(g_host).pin_memory()

    def e2e_step(grad_back):
        a = f_host.to(dev, non_blocking=True).requires_grad_(True)
        b = g_host.to(dev, non_blocking=True).requires_grad_(True)
        y, p, q = ys_h.to(dev, non_blocking=True), lx_h.to(dev, non_blocking=True), ly_h.to(dev, non_blocking=True)
        out = sharded_ctct_simple_loss(a, b, y, p, q, global_batch=G, reduction="mean")
        out.backward()
        if grad_back:
            gf_host.copy_(a.grad, non_blocking=True)
            gg_host.copy_(b.grad, non_blocking=True)
        return float(out.item())

    def timed_e2e(grad_back):
        for _ in range(2):
            e2e_step(grad_back)
        ms, _, _ = timer.timed(lambda: e2e_step(grad_back), e2e_steps)
        return G * e2e_steps / (ms * 1e-3)

    h2d = 4 * (f_host.numel() + g_host.numel() + ys_h.numel() + lx_h.numel() + ly_h.numel())
    variants = {
        "full_copy": {"value": timed_e2e(False), "unit": UNIT, "h2d_bytes_per_step": int(h2d * world),
                      "d2h_bytes_per_step": 4 * world,
                      "note": "f and g copied from pinned host memory every step; gradients stay on the device, loss read back"},
        "full_copy_grad_back": {"value": timed_e2e(True), "unit": UNIT, "h2d_bytes_per_step": int(h2d * world),
                                "d2h_bytes_per_step": int((4 * (f_host.numel() + g_host.numel()) + 4) * world),
                                "note": "as full_copy, and both gradients copied back to pinned host memory"},
    }
    e2e = dict(variants["full_copy"], steps=e2e_steps, variant="full_copy", variants=variants)

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": warm, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": make_config(name, world, args.scaling),
        "clocks": clocks, "e2e": e2e, "gpu_launches": (12 if U1 <= 128 else 13) * args.steps * args.passes * world,
        "passes": pass_stats(per), "roofline": roofline, "kernels": kernels, "step_floor": step_floor,
        "host_enqueue_us_per_step": host_us, "profiled_pass_ms_per_step": ms_profiled / args.steps,
    }
    if graph_ms is not None:
        line["cuda_graph_replay_ms_per_step"] = graph_ms
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        import oracle
        cores = host_cores()
        nb = min(B, 4)
        go = np.full((nb,), 1.0 / G, np.float32)
        t0 = time.perf_counter()
        costs_cpu, _, _ = oracle.simple_loss(f_np[:nb], g_np[:nb], ys[:nb], lx[:nb], ly[:nb], True, go, nthreads=cores)
        dt_s = time.perf_counter() - t0
        with torch.no_grad():
            from warp_ctct_b200 import ctct_simple_loss
            costs_gpu = ctct_simple_loss(f[:nb], g[:nb], ys_t[:nb], lx_t[:nb], ly_t[:nb], reduction="none").cpu().numpy()
        line["cpu_baseline"] = {"value": nb / dt_s, "unit": UNIT, "cores": cores, "kind": "port",
                                "sample": f"the first {nb} of {B} utterances, one pass, {cores} host threads (OpenMP C port); "
                                          f"costs agree with the GPU to "
                                          f"{float(np.abs(costs_cpu - costs_gpu).max() / np.abs(costs_cpu).max()):.1e} rel"}
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        from warp_ctct_b200.sharded import close_scalar_comms
        dist.barrier()
        close_scalar_comms()
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--passes", type=int, default=5, help="timed passes of --steps steps each (median reported)")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    choices = ([w + v for w in sorted(WORKLOADS) for v in ("", "_logits", "_packed", "_logits_packed")]
               + sorted(SIMPLE_WORKLOADS) + ["gather_probe"])
    ap.add_argument("--workload", default="c2", choices=choices)
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"])
    ap.add_argument("--e2e-steps", type=int, default=20)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end (host-resident inputs) measurements")
    ap.add_argument("--no-extra", action="store_true", help="skip the secondary c5 measurement of the default workload")
    args = ap.parse_args()
    args.passes = max(1, args.passes)
    if args.workload == "gather_probe":
        return run_gather_probe(args)
    if args.impl == "reference":
        if args.steps == 200 and "--steps" not in " ".join(sys.argv):
            args.steps, args.warmup = 10, 3
        return run_reference_simple(args) if args.workload in SIMPLE_WORKLOADS else run_reference(args)
    return run_b200_simple(args) if args.workload in SIMPLE_WORKLOADS else run_b200(args)


if __name__ == "__main__":
    sys.exit(main())
