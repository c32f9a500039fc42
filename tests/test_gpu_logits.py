"""GPU parity of ctct_loss_from_logits (log-softmax fused into the loss) against the CPU oracle.

Oracle: log_softmax of the (exactly up-cast) logits in float64, rounded to float32, then the
oracle's float64 evaluation of the reference's lattice and occupancy gradient
(csrc/gather.cu:311-374), the dense scatter autograd performs (warp_ctct/__init__.py:31-33,131) and
the chain rule through log_softmax:  d logits = d - softmax * sum_v d.

Tolerances: costs 1e-5 relative; float32 gradients 1e-4 absolute (measured distance printed);
16-bit gradients one step of the output type + 5e-5.
"""
import numpy as np
import pytest
import torch

import oracle
from util import make_case

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


def _dev(*arrs):
    return [torch.from_numpy(np.ascontiguousarray(a)).to(DEV) for a in arrs]


def oracle_from_logits(x, ys, lx, ly, grad_out):
    """x: float32 logits (N,T,U1,V) as the kernels see them.  Returns (costs, d loss / d logits) in float64."""
    x64 = x.astype(np.float64)
    m = x64.max(-1, keepdims=True)
    m = np.where(np.isfinite(m), m, 0.0)
    lse = m + np.log(np.exp(x64 - m).sum(-1, keepdims=True))
    lp64 = x64 - lse
    lp32 = lp64.astype(np.float32)
    g3 = oracle.collect_units(lp32, ys)
    costs, g64 = oracle.ctct_fwd(g3, ys, lx, ly, True, np.float64)
    g64 = np.where(np.isfinite(costs)[:, None, None, None], g64, 0.0)
    N, T, U1, V = x.shape
    d = np.zeros((N, T, U1, V), np.float64)
    go = np.asarray(grad_out, np.float64)
    for n in range(N):
        for u in range(U1):
            cols = (0, ys[n, u - 1] if u >= 1 else 0, ys[n, u] if u < U1 - 1 else 0)
            for k, c in enumerate(cols):
                d[n, :, u, c] += go[n] * g64[n, :, u, k]
    dl = d - np.exp(lp64) * d.sum(-1, keepdims=True)
    for n in range(N):   # rows outside the valid region carry nothing
        dl[n, lx[n]:] = 0.0
        dl[n, :, ly[n] + 1:] = 0.0
    return costs, dl


@pytest.mark.parametrize("shape,seed,kw", [
    ((3, 12, 5, 8), 1, dict(lx_range=(6, 12), ly_range=(1, 4))),
    ((2, 20, 9, 13), 2, dict(lx_range=(10, 20), ly_range=(2, 8), repeat_prob=0.4)),   # scalar path: V % 4 != 0
    ((4, 33, 17, 130), 3, dict(lx_range=(17, 33), ly_range=(3, 16))),                 # V % 4 == 2
    ((2, 64, 33, 512), 4, dict(lx_range=(40, 64), ly_range=(8, 32))),                 # one 2 KB chunk per row
    ((2, 30, 9, 1100), 5, dict(lx_range=(15, 30), ly_range=(2, 8), repeat_prob=0.3)), # three chunks, ragged tail
    ((2, 9, 4, 36), 6, dict(lx_range=(5, 9), ly_range=(1, 3))),                       # fewer vectors than lanes
])
def test_costs_and_gradient_fp32(W, shape, seed, kw):
    N, T, U1, V = shape
    _, ys, lx, ly = make_case(N, T, U1, V, 1.0, seed, **kw)
    rng = np.random.default_rng(seed)
    x = (2.0 * rng.standard_normal((N, T, U1, V)) + rng.uniform(-5, 5)).astype(np.float32)
    ys[0, :2] = 0   # labels that collide with the blank column
    go = rng.uniform(0.2, 2.0, N).astype(np.float32)
    x_t = torch.from_numpy(x).to(DEV).requires_grad_(True)
    ys_t, lx_t, ly_t, go_t = _dev(ys, lx, ly, go)
    costs = W.ctct_loss_from_logits(x_t, ys_t, lx_t, ly_t, reduction="none")
    costs.backward(go_t)
    c_ref, d_ref = oracle_from_logits(x, ys, lx, ly, go)
    fin = np.isfinite(c_ref)
    c = costs.detach().cpu().numpy()
    assert np.array_equal(np.isposinf(c), ~fin)
    np.testing.assert_allclose(c[fin], c_ref[fin], rtol=1e-5)
    got = x_t.grad.cpu().numpy()
    err = np.abs(got - d_ref).max()
    print(f"\nshape {shape}: max |grad - oracle64| = {err:.2e}")
    assert err < 1e-4
    for n in range(N):
        assert not got[n, lx[n]:].any() and not got[n, :, ly[n] + 1:].any()
    # the same thing through the unfused path of this library: log_softmax by torch, then ctct_loss
    y_t = torch.from_numpy(x).to(DEV).requires_grad_(True)
    W.ctct_loss(y_t.log_softmax(-1), ys_t, lx_t, ly_t, reduction="none").backward(go_t)
    assert (x_t.grad - y_t.grad).abs().max().item() < 1e-4


@pytest.mark.parametrize("dtype,step", [(torch.float16, 2.0 ** -10), (torch.bfloat16, 2.0 ** -7)])
@pytest.mark.parametrize("V", [264, 70])   # 16-byte vectors / scalar path
def test_gradient_16bit(W, dtype, step, V):
    N, T, U1 = 3, 40, 17
    _, ys, lx, ly = make_case(N, T, U1, V, 1.0, 61, lx_range=(20, 40), ly_range=(2, 16), repeat_prob=0.3)
    rng = np.random.default_rng(61)
    x16 = torch.from_numpy((2.0 * rng.standard_normal((N, T, U1, V))).astype(np.float32)).to(dtype)
    x = x16.float().numpy()
    x_t = x16.to(DEV).requires_grad_(True)
    ys_t, lx_t, ly_t = _dev(ys, lx, ly)
    loss = W.ctct_loss_from_logits(x_t, ys_t, lx_t, ly_t, reduction="sum")
    loss.backward()
    assert x_t.grad.dtype == dtype
    c_ref, d_ref = oracle_from_logits(x, ys, lx, ly, np.ones(N))
    assert abs(loss.item() - c_ref.sum()) < 1e-5 * c_ref.sum()
    got = x_t.grad.float().cpu().numpy()
    assert np.all(np.abs(got - d_ref) <= step * np.abs(d_ref) + 5e-5)


def test_reductions_no_grad_and_masked_vocabulary(W):
    N, T, U1, V = 5, 18, 6, 24
    _, ys, lx, ly = make_case(N, T, U1, V, 1.0, 71, lx_range=(9, 18), ly_range=(1, 5))
    rng = np.random.default_rng(71)
    x = rng.standard_normal((N, T, U1, V)).astype(np.float32)
    x[..., 20:] = -np.inf            # vocabulary entries masked out: probability zero, gradient zero
    ys = np.minimum(ys, 19).astype(np.int32)
    c_ref, _ = oracle_from_logits(x, ys, lx, ly, np.ones(N))
    ys_t, lx_t, ly_t = _dev(ys, lx, ly)
    for red, want in (("none", c_ref), (None, c_ref), ("sum", c_ref.sum()), ("mean", c_ref.mean())):
        x_t = torch.from_numpy(x).to(DEV)
        loss = W.ctct_loss_from_logits(x_t, ys_t, lx_t, ly_t, reduction=red)
        np.testing.assert_allclose(loss.cpu().numpy(), want, rtol=1e-5)
        assert not loss.requires_grad
    x_t = torch.from_numpy(x).to(DEV).requires_grad_(True)
    loss = W.ctct_loss_from_logits(x_t, ys_t, lx_t, ly_t, reduction="mean", average_frames=True)
    np.testing.assert_allclose(loss.item(), (c_ref / lx).mean(), rtol=1e-5)
    loss.backward()
    _, d_ref = oracle_from_logits(x, ys, lx, ly, 1.0 / (N * lx))
    got = x_t.grad.cpu().numpy()
    assert not np.isnan(got).any()
    assert np.abs(got - d_ref).max() < 1e-5
    assert not got[..., 20:].any()
    # a shard of a larger batch: 'mean' divides by the global batch
    y_t = torch.from_numpy(x).to(DEV).requires_grad_(True)
    l4 = W.ctct_loss_from_logits(y_t, ys_t, lx_t, ly_t, reduction="mean", average_frames=True, global_batch=4 * N)
    l4.backward()
    assert abs(l4.item() * 4 - loss.item()) < 1e-6 * abs(loss.item())
    assert (y_t.grad * 4 - x_t.grad).abs().max().item() < 1e-6
    # every row of the gradient of a live frame sums to zero (softmax is invariant to a shift of its row)
    assert np.abs(got.sum(-1)).max() < 1e-5


def test_benchmark_shape_from_logits(W):
    """B=32, T=256, U+1=65, V=512 float32 raw logits: three utterances against the oracle, all of
    them against the unfused path of this library (torch.log_softmax + ctct_loss)."""
    N, T, U1, V = 32, 256, 65, 512
    g = torch.Generator(device=DEV).manual_seed(2100)
    x_t = (1.5 * torch.randn((N, T, U1, V), device=DEV, generator=g)).requires_grad_(True)
    rng = np.random.default_rng(2100)
    lx = rng.integers(128, 257, N).astype(np.int32)
    ly = np.minimum(rng.integers(16, 65, N), lx // 2).astype(np.int32)
    ys = rng.integers(1, V, (N, U1 - 1)).astype(np.int32)
    ys_t, lx_t, ly_t = _dev(ys, lx, ly)
    loss = W.ctct_loss_from_logits(x_t, ys_t, lx_t, ly_t, reduction="mean")
    loss.backward()
    grad = x_t.grad
    y_t = x_t.detach().clone().requires_grad_(True)
    loss2 = W.ctct_loss(y_t.log_softmax(-1), ys_t, lx_t, ly_t, reduction="mean")
    loss2.backward()
    assert abs(loss.item() - loss2.item()) <= 1e-5 * abs(loss2.item())
    assert (grad - y_t.grad).abs().max().item() * N < 1e-4
    for n in range(N):
        assert not grad[n, lx[n]:].any().item() and not grad[n, :, ly[n] + 1:].any().item()
    for n in (0, 13, 31):
        sl = slice(n, n + 1)
        c_ref, d_ref = oracle_from_logits(x_t[sl].detach().cpu().numpy(), ys[sl], lx[sl], ly[sl], [1.0 / N])
        err = np.abs(grad[n].cpu().numpy() - d_ref[0]).max() * N
        print(f"\nutterance {n}: max |grad - oracle64| (per unit of upstream gradient) = {err:.2e}")
        assert err < 1e-4


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_padding_cleared_in_the_forward_pass_gives_the_same_gradient(W, dtype, monkeypatch):
    """With the gradient buffer allocated by the forward pass, extra blocks of the lattice launch zero
    its padding rows and the backward kernel writes valid rows only; without, the backward kernel
    writes everything.  Same bits either way, also for a second backward through a retained graph."""
    N, T, U1, V = 5, 37, 12, 72
    _, ys, lx, ly = make_case(N, T, U1, V, 1.0, 91, lx_range=(10, 37), ly_range=(1, 11), repeat_prob=0.2)
    lx[1], ly[2] = 37, 11
    rng = np.random.default_rng(91)
    x = torch.from_numpy(rng.standard_normal((N, T, U1, V)).astype(np.float32)).to(dtype)
    ys_t, lx_t, ly_t = _dev(ys, lx, ly)
    go = torch.tensor([0.5, 2.0, 1.25, 1.0, 0.75], device=DEV)
    grads = {}
    for mode in ("one_pass", "padding_precleared"):
        monkeypatch.setattr(W, "PREZERO", mode == "padding_precleared")
        monkeypatch.setattr(W, "PREZERO_MIN_BYTES", 0)
        for red in ("none", "mean"):
            x_t = x.to(DEV).requires_grad_(True)
            loss = W.ctct_loss_from_logits(x_t, ys_t, lx_t, ly_t, reduction=red, average_frames=True)
            if red == "none":
                # poison what the allocator hands out next, so that stale bytes cannot pass for zeros
                junk = torch.full_like(x_t, 7.0)
                del junk
                loss.backward(go, retain_graph=True)
                first = x_t.grad.clone()
                x_t.grad = None
                loss.backward(go)
                assert torch.equal(first, x_t.grad)
            else:
                loss.backward()
            grads[(mode, red)] = x_t.grad.clone()
    for red in ("none", "mean"):
        assert torch.equal(grads[("one_pass", red)], grads[("padding_precleared", red)]), red
    _, d_ref = oracle_from_logits(x.float().numpy(), ys, lx, ly, go.cpu().numpy() / lx)
    got = grads[("padding_precleared", "none")].float().cpu().numpy()
    tol = 1e-4 if dtype == torch.float32 else 2e-3
    assert np.abs(got - d_ref).max() < tol
    for n in range(N):
        assert not got[n, lx[n]:].any() and not got[n, :, ly[n] + 1:].any()
