"""CPU oracle for the CTC-Transducer loss: TEST INFRASTRUCTURE, not product code.

Thin ctypes/numpy front-end over ``libctct_oracle.so`` (built from ``ctct_oracle.c`` by
``make -C oracle``).  The C file restates the reference project's algorithm and cites the
reference file:line for every function; this module only marshals numpy arrays.

Only ``tests/``, the smoke check and the CPU-baseline leg of ``bench.py`` import this
package.  The product (``warp_ctct_b200``) never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libctct_oracle.so")
_lib = None

FW_SIMPLE, BW_SIMPLE, FW_SHIFT, BW_SHIFT = 0, 1, 2, 3


def build(force: bool = False) -> str:
    """Compile the oracle with gcc (``make -C oracle``); returns the library path."""
    srcs = [os.path.join(_HERE, n) for n in ("ctct_oracle.c", "ctct_oracle_impl.inc", "Makefile")]
    stale = (not os.path.exists(_SO)) or any(
        os.path.exists(s) and os.path.getmtime(s) > os.path.getmtime(_SO) for s in srcs
    )
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B"], check=True, capture_output=True)
    return _SO


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_SO)
    return _lib


def _p(a, t):
    return a.ctypes.data_as(C.POINTER(t))


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def max_threads() -> int:
    return int(lib().oracle_max_threads())


def collect_units(lp, ys, nthreads: int = 0):
    """(N,T,U1,V) float32, (N,U1-1) int -> (N,T,U1,3); ref_ctct.py:223-230."""
    lp, ys = _f32(lp), _i32(ys)
    N, T, U1, V = lp.shape
    out = np.empty((N, T, U1, 3), np.float32)
    rc = lib().oracle_collect_units(_p(lp, C.c_float), _p(ys, C.c_int), N, T, U1, V, _p(out, C.c_float), nthreads)
    assert rc == 0
    return out


def table(g3, ys, which: int, dtype=np.float32):
    """One utterance: g3 (T,U+1,3), ys (U,) -> (table, log-likelihood) in one of ref_ctct.py's layouts."""
    g3, ys = _f32(g3), _i32(ys)
    T, U1, _ = g3.shape
    U = U1 - 1
    assert ys.shape[0] >= U
    rows = T + 1 if which in (FW_SIMPLE, BW_SIMPLE) else T - U + 1
    if dtype == np.float32:
        tab, ll = np.empty((rows, 2 * U + 1), np.float32), C.c_float()
        rc = lib().oracle_table_f32(_p(g3, C.c_float), U1, _p(ys, C.c_int), T, U, which, _p(tab, C.c_float), C.byref(ll))
    else:
        tab, ll = np.empty((rows, 2 * U + 1), np.float64), C.c_double()
        rc = lib().oracle_table_f64(_p(g3, C.c_float), U1, _p(ys, C.c_int), T, U, which, _p(tab, C.c_double), C.byref(ll))
    assert rc == 0, rc
    return tab, ll.value


def ctct_fwd(g3, ys, lx, ly, want_grad: bool = True, dtype=np.float32, nthreads: int = 0):
    """Batch (N,T,U1,3) gathered log-probs -> (costs (N,), grads (N,T,U1,3) or None).

    Restates csrc/binding.cpp:31-100 + csrc/gather.cu:311-374 over ref_ctct.py's band tables."""
    g3, ys, lx, ly = _f32(g3), _i32(ys), _i32(lx), _i32(ly)
    N, T, U1, _ = g3.shape
    ct = C.c_float if dtype == np.float32 else C.c_double
    costs = np.empty((N,), dtype)
    grads = np.empty((N, T, U1, 3), dtype) if want_grad else np.empty((1,), dtype)
    fn = lib().oracle_ctct_fwd_f32 if dtype == np.float32 else lib().oracle_ctct_fwd_f64
    rc = fn(_p(g3, C.c_float), _p(ys, C.c_int), _p(lx, C.c_int), _p(ly, C.c_int), N, T, U1, int(want_grad),
            _p(costs, ct), _p(grads, ct), nthreads)
    assert rc == 0, rc
    return costs, (grads if want_grad else None)


def scatter_dense(grads3, ys, grad_out, V: int, half_round: bool = False, nthreads: int = 0):
    """Dense (N,T,U1,V) gradient autograd builds from the 3-slot gradient (warp_ctct/__init__.py:31-33,131)."""
    grads3, ys, grad_out = _f32(grads3), _i32(ys), _f32(grad_out)
    N, T, U1, _ = grads3.shape
    dense = np.empty((N, T, U1, V), np.float32)
    rc = lib().oracle_scatter_dense(_p(grads3, C.c_float), _p(ys, C.c_int), _p(grad_out, C.c_float), N, T, U1, V,
                                    int(half_round), _p(dense, C.c_float), nthreads)
    assert rc == 0
    return dense


def ctct_loss(lp, ys, lx, ly, grad_out=None, want_grad: bool = True, nthreads: int = 0):
    """Whole path on host memory in fp32: returns (costs, dense grad or None)."""
    lp, ys, lx, ly = _f32(lp), _i32(ys), _i32(lx), _i32(ly)
    N, T, U1, V = lp.shape
    go = _f32(np.ones((N,), np.float32) if grad_out is None else grad_out)
    costs = np.empty((N,), np.float32)
    dense = np.empty((N, T, U1, V), np.float32) if want_grad else None
    fn = lib().oracle_ctct_loss_f32
    fn.argtypes = [C.c_void_p] * 4 + [C.c_int] * 4 + [C.c_void_p] * 3 + [C.c_int]
    rc = fn(lp.ctypes.data, ys.ctypes.data, lx.ctypes.data, ly.ctypes.data, N, T, U1, V, go.ctypes.data,
            costs.ctypes.data, dense.ctypes.data if want_grad else None, nthreads)
    assert rc == 0, rc
    return costs, dense


def round_half(x: float) -> float:
    fn = lib().oracle_round_half
    fn.restype, fn.argtypes = C.c_float, [C.c_float]
    return float(fn(x))


# ----------------------------------------------------------------------------- simple loss

def log_matmul(f, g, dtype=np.float64, nthreads: int = 0):
    """den[b,i,j] = log sum_k exp(f[b,i,k] + g[b,j,k]); csrc/logmatmul.cu:44-146."""
    f, g = _f32(f), _f32(g)
    B, M, K = f.shape
    Nc = g.shape[1]
    out = np.empty((B, M, Nc), dtype)
    if dtype == np.float32:
        rc = lib().oracle_log_matmul_f32(_p(f, C.c_float), _p(g, C.c_float), B, M, Nc, K, _p(out, C.c_float), nthreads)
    else:
        rc = lib().oracle_log_matmul_f64(_p(f, C.c_float), _p(g, C.c_float), B, M, Nc, K, _p(out, C.c_double), nthreads)
    assert rc == 0
    return out


def collect_separate(f, g, ys):
    """ref_ctct.py:206-220: f (N,T,V) -> (N,T,U1); g (N,U1,V) -> (N,U1,3)."""
    f, g, ys = _f32(f), _f32(g), _i32(ys)
    N, T, V = f.shape
    U1 = g.shape[1]
    cf, cg = np.empty((N, T, U1), np.float32), np.empty((N, U1, 3), np.float32)
    rc = lib().oracle_collect_separate(_p(f, C.c_float), _p(g, C.c_float), _p(ys, C.c_int), N, T, U1, V,
                                       _p(cf, C.c_float), _p(cg, C.c_float))
    assert rc == 0
    return cf, cg


def compose_simple(cf, cg, den=None):
    """csrc/simple.cu:20-26: gathered f, g (and den) -> the (N,T,U1,3) log-probs the lattice sees."""
    cf, cg = _f32(cf), _f32(cg)
    N, T, U1 = cf.shape
    g3 = np.empty((N, T, U1, 3), np.float32)
    dp = None
    if den is not None:
        den = _f32(den)
        dp = _p(den, C.c_float)
    rc = lib().oracle_compose_simple(_p(cf, C.c_float), _p(cg, C.c_float), dp, N, T, U1, _p(g3, C.c_float))
    assert rc == 0
    return g3


def simple_reduce(grads3, with_den: bool = True):
    """csrc/binding.cpp:198,209-219: 3-slot grads -> (grad_cf (N,T,U1), grad_cg (N,U1,3), grad_den (N,T,U1))."""
    grads3 = _f32(grads3)
    N, T, U1, _ = grads3.shape
    gcf, gcg = np.empty((N, T, U1), np.float32), np.empty((N, U1, 3), np.float32)
    gden = np.empty((N, T, U1), np.float32) if with_den else None
    rc = lib().oracle_simple_reduce(_p(grads3, C.c_float), N, T, U1, _p(gcf, C.c_float), _p(gcg, C.c_float),
                                    _p(gden, C.c_float) if with_den else None)
    assert rc == 0
    return gcf, gcg, gden


def log_matmul_backward(grad_den, f, g, den, grad_f=None, grad_g=None, nthreads: int = 0):
    """csrc/binding.cpp:251-253 in double; accumulates into grad_f (B,M,K) / grad_g (B,Nc,K) float64."""
    grad_den, f, g, den = _f32(grad_den), _f32(f), _f32(g), _f32(den)
    B, M, K = f.shape
    Nc = g.shape[1]
    if grad_f is None:
        grad_f = np.zeros((B, M, K), np.float64)
    if grad_g is None:
        grad_g = np.zeros((B, Nc, K), np.float64)
    rc = lib().oracle_log_matmul_backward(_p(grad_den, C.c_float), _p(f, C.c_float), _p(g, C.c_float),
                                          _p(den, C.c_float), B, M, Nc, K, _p(grad_f, C.c_double),
                                          _p(grad_g, C.c_double), nthreads)
    assert rc == 0
    return grad_f, grad_g


def simple_loss(f, g, ys, lx, ly, normalized: bool = True, grad_out=None, nthreads: int = 0, dtype=np.float32):
    """ctct_simple_loss on host: returns (costs, grad_f (N,T,V), grad_g (N,U1,V)) as float64 arrays.
    dtype float32 follows the reference's arithmetic (float32 denominator and tables); float64
    evaluates the denominator and the lattice in double (the composed log-probs stay float32).

    Composition of warp_ctct/__init__.py:150-236: den = log_matmul, gathers, lattice on
    f+g-den, reductions, scatter back to the vocabulary, plus the log_matmul backward."""
    f, g, ys, lx, ly = _f32(f), _f32(g), _i32(ys), _i32(lx), _i32(ly)
    N, T, V = f.shape
    U1 = g.shape[1]
    den = log_matmul(f, g, dtype, nthreads).astype(np.float32) if normalized else None
    cf, cg = collect_separate(f, g, ys)
    g3 = compose_simple(cf, cg, den)
    costs, grads3 = ctct_fwd(g3, ys, lx, ly, True, dtype, nthreads)
    go = np.ones((N,), np.float32) if grad_out is None else _f32(grad_out)
    grads3 = (grads3 * go[:, None, None, None]).astype(np.float32)
    gcf, gcg, gden = simple_reduce(grads3, normalized)
    gf = np.zeros((N, T, V), np.float64)
    gg = np.zeros((N, U1, V), np.float64)
    for n in range(N):
        np.add.at(gf[n], (slice(None), 0), gcf[n, :, 0])
        for u in range(1, U1):
            gf[n, :, ys[n, u - 1]] += gcf[n, :, u]
        for u in range(U1):
            gg[n, u, 0] += gcg[n, u, 0]
            gg[n, u, ys[n, u - 1] if u >= 1 else 0] += gcg[n, u, 1]
            gg[n, u, ys[n, u] if u < U1 - 1 else 0] += gcg[n, u, 2]
    if normalized:
        log_matmul_backward(gden, f, g, den, gf, gg, nthreads)
    return costs, gf, gg
