"""The reference's STYLE of CPU path, restated: TEST INFRASTRUCTURE, not product code.

The reference project's only CPU implementation (ref_ctct.py:6-203) evaluates the lattice one cell
at a time in Python, every cell a handful of scalar ``torch.logaddexp`` calls on 0-dim tensors, and
visits only the cells of the band a state can live in (ref_ctct.py:85-87: ``T-U+1`` cells per state).
This module does the same work in the same way -- forward variables, backward variables and the
occupancy gradient of csrc/gather.cu:311-374, per-cell Python loops over torch scalars, band cells
only -- so that the benchmark can time "the reference's own kind of CPU code" on the machine it
runs on.  (The reference's file itself cannot be shipped or read at run time.)  Written in plain
time-synchronous coordinates: alpha[t, s] after t frames, s in [0, 2U].

tests/test_oracle.py pins it to the reference's golden outputs.  Only tests/ and the CPU-baseline
leg of bench.py import it.
"""
from __future__ import annotations

import time

import numpy as np
import torch

NEG_INF = float("-inf")


def _band(t: int, T: int, U: int):
    """States that can be occupied after t frames: reachable from the start and able to reach the end
    (one frame per state change, one label per odd state)."""
    lo = max(0, 2 * U - 2 * (T - t) - 1) if t < T else 2 * U - 1
    hi = min(2 * U, 2 * t - 1) if t > 0 else 0
    return max(lo, 0), hi


def forward_variables(lp: torch.Tensor, ys: torch.Tensor):
    """alpha (T+1, 2U+1) and the log-likelihood; recursion of ref_ctct.py:22-37."""
    T, U1 = lp.shape[:2]
    U = U1 - 1
    S = 2 * U + 1
    alpha = torch.full((T + 1, S), NEG_INF, dtype=lp.dtype)
    alpha[0, 0] = 0.0
    for t in range(1, T + 1):
        lo, hi = _band(t, T, U)
        for s in range(lo, hi + 1):
            u = (s + 1) // 2
            yn = 0 if s % 2 == 0 else int(ys[u - 1])
            acc = alpha[t - 1, s] + lp[t - 1, u, yn]
            if s >= 1:
                acc = torch.logaddexp(acc, alpha[t - 1, s - 1] + lp[t - 1, s // 2, yn])
            if s % 2 == 1 and s > 1 and ys[u - 1] != ys[u - 2]:
                acc = torch.logaddexp(acc, alpha[t - 1, s - 2] + lp[t - 1, u - 1, yn])
            alpha[t, s] = acc
    ll = alpha[T, 2 * U]
    if U >= 1:
        ll = torch.logaddexp(ll, alpha[T, 2 * U - 1])
    return alpha, ll


def backward_variables(lp: torch.Tensor, ys: torch.Tensor):
    """beta (T+1, 2U+1) and the log-likelihood beta[0, 0]; recursion of ref_ctct.py:56-74."""
    T, U1 = lp.shape[:2]
    U = U1 - 1
    S = 2 * U + 1
    beta = torch.full((T + 1, S), NEG_INF, dtype=lp.dtype)
    beta[T, 2 * U] = 0.0
    if U >= 1:
        beta[T, 2 * U - 1] = 0.0
    for t in range(T - 1, -1, -1):
        lo, hi = _band(t, T, U)
        for s in range(lo, hi + 1):
            u = (s + 1) // 2                      # context of state s
            yn = 0 if s % 2 == 0 else int(ys[u - 1])
            acc = beta[t + 1, s] + lp[t, u, yn]   # stay: repeat the label / another blank
            if s + 1 < S:
                if s % 2 == 0:                    # blank 2u -> label 2u+1, emits label u at context u
                    acc = torch.logaddexp(acc, beta[t + 1, s + 1] + lp[t, u, int(ys[u])])
                else:                             # label 2u-1 -> blank 2u, emits blank at context u
                    acc = torch.logaddexp(acc, beta[t + 1, s + 1] + lp[t, u, 0])
            if s % 2 == 1 and s + 2 < S and ys[u] != ys[u - 1]:   # label -> next, different label
                acc = torch.logaddexp(acc, beta[t + 1, s + 2] + lp[t, u, int(ys[u])])
            beta[t, s] = acc
    return beta, beta[0, 0]


def occupancy_gradient(lp: torch.Tensor, ys: torch.Tensor, alpha: torch.Tensor, beta: torch.Tensor, ll: torch.Tensor):
    """d cost / d (the three gathered log-probs of every (t, u)): (T, U+1, 3), csrc/gather.cu:311-374."""
    T, U1 = lp.shape[:2]
    U = U1 - 1
    grad = torch.zeros((T, U1, 3), dtype=lp.dtype)
    for t in range(T):
        for u in range(U1):
            b = 2 * u                                  # blank state of context u
            g0 = torch.exp(alpha[t, b] + lp[t, u, 0] + beta[t + 1, b] - ll)
            g1 = torch.zeros(())
            g2 = torch.zeros(())
            if u >= 1:                                 # label state 2u-1
                l = 2 * u - 1
                g0 = g0 + torch.exp(alpha[t, l] + lp[t, u, 0] + beta[t + 1, b] - ll)
                g1 = torch.exp(alpha[t, l] + lp[t, u, int(ys[u - 1])] + beta[t + 1, l] - ll)
            if u < U:
                nxt = 2 * u + 1
                p = lp[t, u, int(ys[u])]
                g2 = torch.exp(alpha[t, b] + p + beta[t + 1, nxt] - ll)
                if u >= 1 and ys[u] != ys[u - 1]:
                    g2 = g2 + torch.exp(alpha[t, 2 * u - 1] + p + beta[t + 1, nxt] - ll)
            grad[t, u, 0] = -g0
            grad[t, u, 1] = -g1
            grad[t, u, 2] = -g2
    return grad


def loss_and_gradient(lp, ys):
    """One utterance, trimmed to its lengths: lp (T, U+1, V), ys (U,) -> (cost, gradient (T, U+1, 3))."""
    lp = torch.as_tensor(lp)
    ys = torch.as_tensor(ys)
    alpha, _ = forward_variables(lp, ys)
    beta, ll = backward_variables(lp, ys)
    return float(-ll), occupancy_gradient(lp, ys, alpha, beta, ll)


def _timed_one(job):
    lp, ys = job
    torch.set_num_threads(1)
    t0 = time.perf_counter()
    loss_and_gradient(lp, ys)
    return time.perf_counter() - t0


def time_utterances(lp, ys, lx, ly, processes: int = 1, budget_s: float = 60.0):
    """Seconds each of the given utterances takes (forward + backward variables + gradient) on one core,
    run `processes` at a time in spawned single-threaded worker processes.  lp (N,T,U1,V) float32."""
    import multiprocessing as mp
    jobs = []
    for n in range(len(lx)):
        Tn, Un = int(lx[n]), int(ly[n])
        jobs.append((np.ascontiguousarray(lp[n, :Tn, :Un + 1]), np.ascontiguousarray(ys[n, :Un]).astype(np.int64)))
    if processes <= 1:
        return [_timed_one(j) for j in jobs]
    ctx = mp.get_context("spawn")
    with ctx.Pool(processes) as pool:
        res = pool.map_async(_timed_one, jobs)
        try:
            return list(res.get(timeout=max(budget_s, 1.0) * 6))
        except mp.TimeoutError:
            return []
