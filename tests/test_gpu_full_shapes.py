"""Parity at the FULL shapes of the benchmark configurations, through the public API.

The small-shape tests pin the arithmetic; these run every kernel at the sizes the benchmark uses
(nine lattice warps per direction, four row tiles x 64 k-blocks of the tensor-core GEMM, tensors
beyond 2^32 elements, more than 2^29 rows) and check a sample of utterances against the CPU
oracle plus what does not depend on size: one emission per frame and zero padding.

Tolerances: float32 costs 1e-5 relative; float32 gradients 1e-4 absolute (+ the float32 oracle's
own distance to its float64 evaluation, printed); float16 gradients one float16 step of the
oracle value + 5e-5.
"""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def W():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import warp_ctct_b200
    from warp_ctct_b200 import _lib
    _lib.lib()
    return warp_ctct_b200


@pytest.fixture(autouse=True)
def _release_device_memory():
    yield
    if torch.cuda.is_available():
        torch.cuda.empty_cache()


def _dev(*arrs):
    return [torch.from_numpy(np.ascontiguousarray(a)).to(DEV) for a in arrs]


def _lengths(seed, N, U1, V, lxr, lyr, cap_half):
    rng = np.random.default_rng(seed)
    lx = rng.integers(lxr[0], lxr[1] + 1, N).astype(np.int32)
    ly = rng.integers(lyr[0], lyr[1] + 1, N).astype(np.int32)
    if cap_half:
        ly = np.minimum(ly, lx // 2).astype(np.int32)
    ly = np.minimum(ly, lx).astype(np.int32)
    ys = rng.integers(1, V, (N, U1 - 1)).astype(np.int32)
    return lx, ly, ys


def _joint(N, T, U1, V, sigma, dtype, seed, chunk=8):
    """log_softmax(sigma * N(0,1)) in `dtype`, generated on the device a few utterances at a time."""
    gen = torch.Generator(device=DEV).manual_seed(seed)
    out = torch.empty((N, T, U1, V), dtype=dtype, device=DEV)
    for n0 in range(0, N, chunk):
        n1 = min(N, n0 + chunk)
        out[n0:n1] = (sigma * torch.randn((n1 - n0, T, U1, V), device=DEV, generator=gen)).log_softmax(-1).to(dtype)
    return out


def _check_standard_loss(W, lp_t, ys, lx, ly, sample, half):
    """ctct_loss fwd+bwd on the whole batch; utterances in `sample` against the oracle, all of them
    against the size-independent properties."""
    N, T, U1, V = lp_t.shape
    ys_t, lx_t, ly_t = _dev(ys, lx, ly)
    lp_t.requires_grad_(True)
    costs = W.ctct_loss(lp_t, ys_t, lx_t, ly_t, reduction="none")
    costs.sum().backward()
    grad = lp_t.grad
    assert grad.dtype == lp_t.dtype and grad.shape == lp_t.shape
    per_frame = -torch.sum(grad, dim=(2, 3), dtype=torch.float32).cpu().numpy()
    for n in range(N):
        # each float16 value carries up to 2^-11 relative rounding; a frame sums <= 3 * (U+1) of them
        np.testing.assert_allclose(per_frame[n, :lx[n]], 1.0, atol=2e-3 if half else 5e-5)
        assert not per_frame[n, lx[n]:].any()
        assert not grad[n, lx[n]:].any().item() and not grad[n, :, ly[n] + 1:].any().item()
    assert int((grad != 0).sum().item()) <= 3 * int((lx.astype(np.int64) * (ly + 1)).sum())
    c_gpu = costs.detach().cpu().numpy()
    assert np.isfinite(c_gpu).all()
    for n in sample:
        lp_n = lp_t[n:n + 1].detach().float().cpu().numpy()   # exact upcast: what the kernels see
        sl = (ys[n:n + 1], lx[n:n + 1], ly[n:n + 1])
        c32, d32 = oracle.ctct_loss(lp_n, *sl)
        g3 = oracle.collect_units(lp_n, sl[0])
        c64, g64 = oracle.ctct_fwd(g3, *sl, True, np.float64)
        d64 = oracle.scatter_dense(g64.astype(np.float32), sl[0], np.ones(1, np.float32), V, half_round=half)
        assert abs(c_gpu[n] - c32[0]) <= 1e-5 * c32[0], (n, c_gpu[n], c32[0])
        assert abs(c_gpu[n] - c64[0]) <= 1e-5 * c64[0], (n, c_gpu[n], c64[0])
        got = grad[n].float().cpu().numpy()
        own32 = float(np.abs(d32[0] - oracle.scatter_dense(g64.astype(np.float32), sl[0], np.ones(1, np.float32), V)[0]).max())
        e64 = np.abs(got - d64[0])
        e32 = np.abs(got - d32[0])
        print(f"\nutterance {n}: lx {lx[n]}, ly {ly[n]}: |gpu - oracle64| = {e64.max():.2e}, "
              f"|gpu - oracle32| = {e32.max():.2e}, |oracle32 - oracle64| = {own32:.2e}")
        if half:
            # one float16 step of the value, plus the float32 bound on the value before rounding
            assert np.all(e64 <= 2.0 ** -10 * np.abs(d64[0]) + 5e-5)
            assert np.all(e32 <= 2.0 ** -10 * np.abs(d32[0]) + 1e-4 + own32)
        else:
            assert e64.max() < 5e-5
            assert e32.max() < 1e-4 + own32
    return c_gpu


def test_config3_fp16_T512_U129_V1024(W):
    """B=16, T=512, U+1=129, V=1024, float16 in, float32 accumulation: nine warps per direction."""
    N, T, U1, V = 16, 512, 129, 1024
    lx, ly, ys = _lengths(3000, N, U1, V, (256, 512), (32, 128), False)
    lx[0], ly[0] = T, U1 - 1                         # one utterance fills the whole tensor
    lp_t = _joint(N, T, U1, V, 2.0, torch.float16, 3000)
    _check_standard_loss(W, lp_t, ys, lx, ly, sample=(0, 15), half=True)


def test_config5_shard_fp16_T400_U101_V1024(W):
    """One rank's share (32 utterances) of the B=256 sharded configuration."""
    N, T, U1, V = 32, 400, 101, 1024
    lx, ly, ys = _lengths(5000, N, U1, V, (100, 400), (10, 100), True)
    lp_t = _joint(N, T, U1, V, 2.0, torch.float16, 5000)
    _check_standard_loss(W, lp_t, ys, lx, ly, sample=(0, 31), half=True)


def test_joint_tensor_beyond_2_to_32_elements(W):
    """(104,400,101,1024) float16 = 4.30e9 elements (8.6 GB, and as large a gradient): row offsets
    of the gather, the clearing blocks and the patch kernel exceed 32 bits for the last utterances,
    which is where the sample is taken."""
    N, T, U1, V = 104, 400, 101, 1024
    assert N * T * U1 * V > 2 ** 32
    lx, ly, ys = _lengths(5100, N, U1, V, (100, 400), (10, 100), True)
    lx[N - 1], ly[N - 1] = T, U1 - 1
    lp_t = _joint(N, T, U1, V, 2.0, torch.float16, 5100)
    _check_standard_loss(W, lp_t, ys, lx, ly, sample=(0, N - 2, N - 1), half=True)


def test_more_than_2_to_29_rows_takes_the_64_bit_gather(W):
    """4200 x 500 x 257 = 5.4e8 rows: the gathered records number more than 2^31 floats, so the
    gather runs with 64-bit element indices.  Forward only (no tables), V = 4 keeps the joint
    tensor at 4.3 GB; costs of utterances across the whole batch against the oracle."""
    from warp_ctct_b200 import _lib
    lib = _lib.lib()
    N, T, U1, V = 4200, 500, 257, 4
    assert N * T * U1 * 4 >= 2 ** 31
    lx, ly, ys = _lengths(5200, N, U1, V, (400, 500), (20, 100), False)
    lx[N - 1], ly[N - 1] = T, 120
    lp_t = _joint(N, T, U1, V, 1.0, torch.float16, 5200, chunk=256)
    ys_t, lx_t, ly_t = _dev(ys, lx, ly)
    dev = torch.device(DEV)
    costs = torch.full((N,), float("nan"), device=dev)
    ws = _lib.workspace(N, T, U1, False, dev)
    rc = lib.ctct_b200_loss_forward(lp_t.data_ptr(), _lib.dtype_code(lp_t.dtype), ys_t.data_ptr(), lx_t.data_ptr(),
                                    ly_t.data_ptr(), N, T, U1, V, 0, costs.data_ptr(), None, ws.data_ptr(), ws.numel(),
                                    _lib.stream_ptr(dev))
    _lib.check(rc, "loss_forward")
    torch.cuda.synchronize()
    c_gpu = costs.cpu().numpy()
    assert not np.isnan(c_gpu).any()
    for n in (0, 1, N // 2, 4093, N - 2, N - 1):
        lp_n = lp_t[n:n + 1].float().cpu().numpy()
        c64, _ = oracle.ctct_fwd(oracle.collect_units(lp_n, ys[n:n + 1]), ys[n:n + 1], lx[n:n + 1], ly[n:n + 1],
                                 False, np.float64)
        if np.isfinite(c64[0]):
            assert abs(c_gpu[n] - c64[0]) <= 1e-5 * c64[0], (n, c_gpu[n], c64[0])
        else:   # more adjacent repeats than spare frames: no alignment
            assert np.isposinf(c_gpu[n])


def test_config4_simple_loss_T500_U101_V4096_on_tensor_cores(W):
    """ctct_simple_loss at B=32, T=500, U+1=101, V=4096: four row tiles x 64 k-blocks in the forward
    GEMM, the fused backward kernel over 64 vocabulary slabs.  Two utterances against the float64
    oracle; the status words must say that the tensor-core results were used."""
    from warp_ctct_b200 import _lib
    N, T, U1, V = 32, 500, 101, 4096
    rng = np.random.default_rng(4000)
    f = rng.standard_normal((N, T, V), dtype=np.float32)
    g = rng.standard_normal((N, U1, V), dtype=np.float32)
    lx, ly, ys = _lengths(4000, N, U1, V, (250, 500), (25, 100), False)
    lx[0], ly[0] = T, U1 - 1
    f_t, g_t = [t.requires_grad_(True) for t in _dev(f, g)]
    ys_t, lx_t, ly_t = _dev(ys, lx, ly)
    go = rng.uniform(0.5, 1.5, N).astype(np.float32)
    costs = W.ctct_simple_loss(f_t, g_t, ys_t, lx_t, ly_t, reduction="none")
    tc_ws = costs.grad_fn.saved_tensors[7]
    assert tc_ws.numel() > 0, "the tensor-core workspace must exist at this shape"
    costs.backward(torch.from_numpy(go).to(DEV), retain_graph=True)
    torch.cuda.synchronize()
    off = _lib.lib().ctct_b200_log_matmul_tc_flags_offset(N, T, U1, V)
    flags = tc_ws[off:off + 16].view(torch.int32).cpu().numpy()
    assert not flags.any(), f"exact fall-back kernels produced the result: flags {flags}"
    c_gpu = costs.detach().cpu().numpy()
    gf, gg = f_t.grad.cpu().numpy(), g_t.grad.cpu().numpy()
    for n in range(N):
        assert not gf[n, lx[n]:].any() and not gg[n, ly[n] + 1:].any()
    for n in (0, 31):
        sl = slice(n, n + 1)
        c_ref, gf_ref, gg_ref = oracle.simple_loss(f[sl], g[sl], ys[sl], lx[sl], ly[sl], True, go[sl], dtype=np.float64)
        assert abs(c_gpu[n] - c_ref[0]) <= 1e-5 * c_ref[0], (n, c_gpu[n], c_ref[0])
        ef = np.abs(gf[n] - gf_ref[0]) - 2e-5 * np.abs(gf_ref[0])
        eg = np.abs(gg[n] - gg_ref[0]) - 2e-5 * np.abs(gg_ref[0])
        print(f"\nutterance {n}: cost {c_gpu[n]:.4f} (oracle {c_ref[0]:.4f}), max |grad_f - oracle| = "
              f"{np.abs(gf[n] - gf_ref[0]).max():.2e}, |grad_g - oracle| = {np.abs(gg[n] - gg_ref[0]).max():.2e}")
        assert ef.max() < 1e-4 and eg.max() < 1e-4
