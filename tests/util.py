"""Seeded synthetic inputs shared by the tests (shapes and distributions of the benchmark configs)."""
import numpy as np


def log_softmax(x):
    x = x - x.max(-1, keepdims=True)
    return (x - np.log(np.exp(x).sum(-1, keepdims=True))).astype(np.float32)


def make_case(N, T, U1, V, sigma=1.0, seed=0, lx_range=None, ly_range=None, cap_half=False, repeat_prob=0.0):
    """log_probs (N,T,U1,V) float32 = log_softmax(sigma * randn), labels in [1, V), ragged lengths."""
    rng = np.random.default_rng(seed)
    lp = log_softmax(sigma * rng.standard_normal((N, T, U1, V), dtype=np.float32))
    ys = rng.integers(1, V, (N, U1 - 1)).astype(np.int32)
    if repeat_prob > 0:
        for n in range(N):
            for u in range(1, U1 - 1):
                if rng.random() < repeat_prob:
                    ys[n, u] = ys[n, u - 1]
    lx_lo, lx_hi = lx_range or (T, T)
    ly_lo, ly_hi = ly_range or (U1 - 1, U1 - 1)
    lx = rng.integers(lx_lo, lx_hi + 1, N).astype(np.int32)
    ly = rng.integers(ly_lo, ly_hi + 1, N).astype(np.int32)
    if cap_half:
        ly = np.minimum(ly, np.maximum(lx // 2, 1)).astype(np.int32)
    ly = np.minimum(ly, lx).astype(np.int32)
    lx[0] = lx_hi  # one utterance uses every frame of the tensor
    ly[0] = min(ly_hi, lx[0] // 2 if cap_half else lx[0])
    return lp, ys, lx, ly
