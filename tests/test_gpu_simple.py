"""GPU parity of the log-add joiner loss (ctct_simple_loss), of the log-semiring matmul and of
the reference's auxiliary classes; every call goes through the C ABI and is checked against the
CPU oracle.  Tolerances: costs 1e-5 relative, gradients 1e-4 absolute (the oracle evaluates the
denominator's backward in float64)."""
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


def _dev(*arrs):
    return [torch.from_numpy(np.ascontiguousarray(a)).to(DEV) for a in arrs]


def _case(N, T, U1, V, seed, lx_range, ly_range, scale=1.0, repeat_prob=0.0):
    rng = np.random.default_rng(seed)
    f = (scale * rng.standard_normal((N, T, V))).astype(np.float32)
    g = (scale * rng.standard_normal((N, U1, V))).astype(np.float32)
    ys = rng.integers(1, V, (N, U1 - 1)).astype(np.int32)
    for n in range(N):
        for u in range(1, U1 - 1):
            if rng.random() < repeat_prob:
                ys[n, u] = ys[n, u - 1]
    lx = rng.integers(lx_range[0], lx_range[1] + 1, N).astype(np.int32)
    ly = np.minimum(rng.integers(ly_range[0], ly_range[1] + 1, N), lx).astype(np.int32)
    lx[0] = T
    return f, g, ys, lx, ly


# ------------------------------------------------------------------------------ log_matmul

@pytest.mark.parametrize("B,M,N,K", [(2, 7, 5, 9), (3, 33, 17, 130), (2, 64, 101, 513), (1, 50, 40, 4096)])
def test_log_matmul_matches_oracle(W, B, M, N, K):
    from warp_ctct_b200.simple import log_matmul
    rng = np.random.default_rng(B * 1000 + K)
    f = (2.0 * rng.standard_normal((B, M, K))).astype(np.float32)
    g = (2.0 * rng.standard_normal((B, N, K))).astype(np.float32)
    want = oracle.log_matmul(f, g, np.float64)
    f_t, g_t = _dev(f, g)
    got = log_matmul(f_t, g_t.transpose(1, 2))                 # the strided view the reference passes
    np.testing.assert_allclose(got.cpu().numpy(), want, rtol=0, atol=2e-5)
    got2 = log_matmul(f_t, g_t.transpose(1, 2).contiguous())   # plain (B,K,N) layout
    np.testing.assert_allclose(got2.cpu().numpy(), want, rtol=0, atol=2e-5)


@pytest.mark.parametrize("B,M,N,K,scale", [(2, 130, 70, 256, 1.0), (3, 33, 17, 64, 2.0), (1, 257, 101, 4096, 1.0),
                                           (2, 128, 128, 520, 3.0), (1, 300, 260, 136, 1.0)])
def test_log_matmul_tensor_core_matches_oracle(W, B, M, N, K, scale):
    """tcgen05 path: bf16 hi+lo operands, fp32 accumulation; the result is held to the float64 oracle."""
    from warp_ctct_b200.simple import log_matmul, log_matmul_tc
    rng = np.random.default_rng(B * 7 + K)
    f = (scale * rng.standard_normal((B, M, K))).astype(np.float32)
    g = (scale * rng.standard_normal((B, N, K))).astype(np.float32)
    f[0, 1, :] = -np.inf                       # dead row -> -inf outputs
    want = oracle.log_matmul(f, g, np.float64)
    f_t, g_t = _dev(f, g)
    got = log_matmul_tc(f_t, g_t).cpu().numpy()
    assert np.all(np.isneginf(got[0, 1])) and np.all(np.isneginf(want[0, 1]))
    fin = np.isfinite(want)
    np.testing.assert_allclose(got[fin], want[fin], rtol=1e-6, atol=5e-6)
    exact = log_matmul(f_t, g_t.transpose(1, 2)).cpu().numpy()
    np.testing.assert_allclose(got[fin], exact[fin], rtol=0, atol=2e-5)


def test_log_matmul_tensor_core_falls_back_on_wide_range(W):
    """Rows whose maxima sit at different k and are > 100 nats above the rest: the max-shifted
    product underflows, the kernel notices and the exact kernel recomputes in the same call."""
    from warp_ctct_b200.simple import log_matmul_tc
    rng = np.random.default_rng(3)
    B, M, N, K = 1, 40, 30, 128
    f = rng.standard_normal((B, M, K)).astype(np.float32)
    g = rng.standard_normal((B, N, K)).astype(np.float32)
    f[0, 5, 3] += 300.0
    g[0, 7, 90] += 300.0
    want = oracle.log_matmul(f, g, np.float64)
    got = log_matmul_tc(*_dev(f, g)).cpu().numpy()
    np.testing.assert_allclose(got, want, rtol=2e-6, atol=2e-5)


def test_log_matmul_extreme_values(W):
    from warp_ctct_b200.simple import log_matmul
    rng = np.random.default_rng(5)
    f = (30.0 * rng.standard_normal((2, 9, 40))).astype(np.float32)   # ~ +-100 nats of range per row
    g = (30.0 * rng.standard_normal((2, 6, 40))).astype(np.float32)
    f[0, 0, :] = -np.inf                       # a row of zeros in probability space
    f[1, 2, :20] = -np.inf
    g[0, 1, 3] = 5000.0                        # exp overflows float32, the log-space result must not
    want = oracle.log_matmul(f, g, np.float64)
    got = log_matmul(*[t for t in (_dev(f)[0], _dev(g)[0].transpose(1, 2))]).cpu().numpy()
    assert np.all(np.isneginf(got[0, 0])) and np.all(np.isneginf(want[0, 0]))
    fin = np.isfinite(want)
    np.testing.assert_allclose(got[fin], want[fin], rtol=2e-6, atol=2e-5)
    with pytest.raises(RuntimeError, match="Float tensor"):
        log_matmul(_dev(f)[0].half(), _dev(g)[0].transpose(1, 2))
    with pytest.raises(RuntimeError, match="invalid sizes"):
        log_matmul(_dev(f)[0], _dev(g)[0])


def test_log_matmul_backward_signed_grad(W):
    from warp_ctct_b200.simple import log_matmul, log_matmul_backward
    rng = np.random.default_rng(8)
    B, M, N, K = 2, 20, 9, 70
    f = rng.standard_normal((B, M, K)).astype(np.float32)
    g = rng.standard_normal((B, N, K)).astype(np.float32)
    go = rng.standard_normal((B, M, N)).astype(np.float32)    # both signs, as a standalone op may see
    f_t, g_t, go_t = _dev(f, g, go)
    rhs = g_t.transpose(1, 2)
    res = log_matmul(f_t, rhs)
    gl, gr = log_matmul_backward(go_t, f_t, rhs, res, [True, True])
    assert gl.shape == (B, M, K) and gr.shape == (B, K, N)
    wl, wr = oracle.log_matmul_backward(go, f, g, res.cpu().numpy())
    np.testing.assert_allclose(gl.cpu().numpy(), wl, atol=2e-5)
    np.testing.assert_allclose(gr.transpose(1, 2).cpu().numpy(), wr, atol=2e-5)
    gl2, gr2 = log_matmul_backward(go_t, f_t, rhs, res, [False, True])
    assert gl2 is None and torch.equal(gr2, gr)
    assert log_matmul_backward(None, f_t, rhs, res, [True, True]) == (None, None)


def test_logmmexp_autograd_matches_logsumexp(W):
    rng = np.random.default_rng(9)
    f = torch.from_numpy(rng.standard_normal((2, 11, 30)).astype(np.float32)).to(DEV)
    g = torch.from_numpy(rng.standard_normal((2, 6, 30)).astype(np.float32)).to(DEV)
    w = torch.from_numpy(rng.standard_normal((2, 11, 6)).astype(np.float32)).to(DEV)
    a, b = f.clone().requires_grad_(True), g.clone().requires_grad_(True)
    (W.LogMMExp.apply(a, b.transpose(1, 2), True, True) * w).sum().backward()
    c, d = f.double().requires_grad_(True), g.double().requires_grad_(True)
    (torch.logsumexp(c[:, :, None, :] + d[:, None, :, :], -1) * w.double()).sum().backward()
    np.testing.assert_allclose(a.grad.cpu().numpy(), c.grad.cpu().numpy(), atol=2e-5)
    np.testing.assert_allclose(b.grad.cpu().numpy(), d.grad.cpu().numpy(), atol=2e-5)


@pytest.mark.parametrize("B,M,N,K", [(2, 150, 70, 128), (1, 40, 140, 264)])
def test_logmmexp_autograd_on_tensor_cores(W, B, M, N, K):
    """The reference's composition LogMMExp(f, g^T) takes the tensor-core kernels in both directions;
    signed upstream gradients, checked against float64 logsumexp."""
    from warp_ctct_b200.simple import _tc_operands
    rng = np.random.default_rng(K)
    f = torch.from_numpy(rng.standard_normal((B, M, K)).astype(np.float32)).to(DEV)
    g = torch.from_numpy(rng.standard_normal((B, N, K)).astype(np.float32)).to(DEV)
    w = torch.from_numpy(rng.standard_normal((B, M, N)).astype(np.float32)).to(DEV)
    a, b = f.clone().requires_grad_(True), g.clone().requires_grad_(True)
    assert _tc_operands(a, b.transpose(1, 2)) is not None
    out = W.LogMMExp.apply(a, b.transpose(1, 2), True, True)
    (out * w).sum().backward()
    c, d = f.double().requires_grad_(True), g.double().requires_grad_(True)
    ref = torch.logsumexp(c[:, :, None, :] + d[:, None, :, :], -1)
    (ref * w.double()).sum().backward()
    np.testing.assert_allclose(out.detach().cpu().numpy(), ref.detach().cpu().numpy(), rtol=1e-6, atol=5e-6)
    np.testing.assert_allclose(a.grad.cpu().numpy(), c.grad.cpu().numpy(), atol=3e-5, rtol=2e-5)
    np.testing.assert_allclose(b.grad.cpu().numpy(), d.grad.cpu().numpy(), atol=3e-5, rtol=2e-5)
    # only one side tracked
    a2 = f.clone().requires_grad_(True)
    (W.LogMMExp.apply(a2, g.transpose(1, 2), True, False) * w).sum().backward()
    np.testing.assert_allclose(a2.grad.cpu().numpy(), c.grad.cpu().numpy(), atol=3e-5, rtol=2e-5)


# ------------------------------------------------------------------------------ the loss

@pytest.mark.parametrize("shape,seed,kw", [
    ((2, 10, 5, 12), 1, dict(lx_range=(6, 10), ly_range=(1, 4))),
    ((4, 25, 9, 40), 2, dict(lx_range=(12, 25), ly_range=(2, 8), repeat_prob=0.3)),
    ((3, 40, 17, 130), 3, dict(lx_range=(20, 40), ly_range=(4, 16))),
    ((2, 30, 34, 67), 4, dict(lx_range=(30, 30), ly_range=(20, 28))),
    ((2, 60, 21, 4096), 5, dict(lx_range=(30, 60), ly_range=(5, 20))),   # vocabulary of the benchmark config
    # shapes the tensor-core path takes (V % 8 == 0, V >= 64): more than one tile / chunk / k-block each way
    ((3, 140, 70, 256), 6, dict(lx_range=(70, 140), ly_range=(30, 69))),
    ((2, 33, 131, 64), 7, dict(lx_range=(33, 33), ly_range=(10, 30))),
    ((2, 260, 9, 72), 8, dict(lx_range=(100, 260), ly_range=(3, 8), repeat_prob=0.3)),
])
@pytest.mark.parametrize("normalized", [True, False])
def test_simple_loss_costs_and_gradients(W, shape, seed, kw, normalized):
    N, T, U1, V = shape
    f, g, ys, lx, ly = _case(N, T, U1, V, seed, **kw)
    go = np.random.default_rng(seed).uniform(0.3, 1.5, N).astype(np.float32)
    f_t, g_t = [t.requires_grad_(True) for t in _dev(f, g)]
    ys_t, lx_t, ly_t, go_t = _dev(ys, lx, ly, go)
    costs = W.ctct_simple_loss(f_t, g_t, ys_t, lx_t, ly_t, reduction="none", normalized=normalized)
    costs.backward(go_t)
    c_ref, gf_ref, gg_ref = oracle.simple_loss(f, g, ys, lx, ly, normalized, go, dtype=np.float64)
    c32, gf32, gg32 = oracle.simple_loss(f, g, ys, lx, ly, normalized, go, dtype=np.float32)
    assert np.isfinite(c_ref).all()
    np.testing.assert_allclose(costs.detach().cpu().numpy(), c_ref, rtol=1e-5)
    np.testing.assert_allclose(costs.detach().cpu().numpy(), c32, rtol=1e-5)
    # the float32 restatement differs from its own float64 evaluation by up to 1e-4 * (frames summed)
    # in grad_g (the noise floor of the reference arithmetic); the kernels are held to the float64 one
    assert np.abs(gf32 - gf_ref).max() < 5e-3 and np.abs(gg32 - gg_ref).max() < 2e-4 * T
    # entries of grad_f / grad_g are sums of up to T*(U+1) occupancies (|value| up to ~T), so the
    # 1e-4 absolute bound on a single occupancy becomes 1e-4 + 2e-5 relative on the sums
    np.testing.assert_allclose(f_t.grad.cpu().numpy(), gf_ref, atol=1e-4, rtol=2e-5)
    np.testing.assert_allclose(g_t.grad.cpu().numpy(), gg_ref, atol=1e-4, rtol=2e-5)
    for n in range(N):   # nothing flows into padding frames / contexts
        assert not f_t.grad[n, lx[n]:].any().item() and not g_t.grad[n, ly[n] + 1:].any().item()


def test_simple_loss_wide_range_falls_back_to_exact_kernels(W):
    """A frame and a context whose maxima sit at different vocabulary entries, 300 nats above the
    rest: the max-shifted sums underflow, and both the denominator and its gradient must come from
    the exact kernels inside the same calls."""
    N, T, U1, V = 2, 24, 7, 128
    f, g, ys, lx, ly = _case(N, T, U1, V, 21, (16, 24), (2, 6))
    f[0, 5, 3] += 300.0
    g[0, 2, 90] += 300.0
    f_t, g_t = [t.requires_grad_(True) for t in _dev(f, g)]
    ys_t, lx_t, ly_t = _dev(ys, lx, ly)
    costs = W.ctct_simple_loss(f_t, g_t, ys_t, lx_t, ly_t, reduction="none")
    costs.sum().backward()
    c_ref, gf_ref, gg_ref = oracle.simple_loss(f, g, ys, lx, ly, True, dtype=np.float64)
    np.testing.assert_allclose(costs.detach().cpu().numpy(), c_ref, rtol=1e-5)
    np.testing.assert_allclose(f_t.grad.cpu().numpy(), gf_ref, atol=1e-4, rtol=2e-5)
    np.testing.assert_allclose(g_t.grad.cpu().numpy(), gg_ref, atol=1e-4, rtol=2e-5)


def test_simple_loss_equals_standard_loss_on_the_joint(W):
    N, T, U1, V = 3, 22, 8, 50
    f, g, ys, lx, ly = _case(N, T, U1, V, 11, (10, 22), (2, 7))
    f_t, g_t, ys_t, lx_t, ly_t = _dev(f, g, ys, lx, ly)
    a, b = f_t.clone().requires_grad_(True), g_t.clone().requires_grad_(True)
    W.ctct_simple_loss(a, b, ys_t, lx_t, ly_t, reduction="mean", average_frames=True).backward()
    c, d = f_t.clone().requires_grad_(True), g_t.clone().requires_grad_(True)
    joint = (c[:, :, None, :] + d[:, None, :, :]).log_softmax(-1)
    W.ctct_loss(joint, ys_t, lx_t, ly_t, reduction="mean", average_frames=True).backward()
    assert (a.grad - c.grad).abs().max().item() < 2e-5 and (b.grad - d.grad).abs().max().item() < 2e-5
    # un-normalised: the raw sum is the log-prob
    a2, b2 = f_t.clone().requires_grad_(True), g_t.clone().requires_grad_(True)
    l1 = W.ctct_simple_loss(a2, b2, ys_t, lx_t, ly_t, reduction="sum", normalized=False)
    c2, d2 = f_t.clone().requires_grad_(True), g_t.clone().requires_grad_(True)
    l2 = W.ctct_loss(c2[:, :, None, :] + d2[:, None, :, :], ys_t, lx_t, ly_t, reduction="sum")
    l1.backward()
    l2.backward()
    assert abs(l1.item() - l2.item()) < 1e-5 * abs(l2.item())
    assert (a2.grad - c2.grad).abs().max().item() < 2e-5 and (b2.grad - d2.grad).abs().max().item() < 2e-5


def test_simple_loss_tracks_only_what_requires_grad(W):
    N, T, U1, V = 2, 12, 5, 20
    f, g, ys, lx, ly = _case(N, T, U1, V, 13, (8, 12), (1, 4))
    f_t, g_t, ys_t, lx_t, ly_t = _dev(f, g, ys, lx, ly)
    a = f_t.clone().requires_grad_(True)
    loss = W.ctct_simple_loss(a, g_t, ys_t, lx_t, ly_t)
    loss.backward()
    assert a.grad is not None and g_t.grad is None
    with torch.no_grad():
        l0 = W.ctct_simple_loss(a, g_t, ys_t, lx_t, ly_t)
    assert not l0.requires_grad and abs(l0.item() - loss.item()) < 1e-6 * abs(loss.item())
    # half inputs are up-cast like the reference does with .float()
    l16 = W.ctct_simple_loss(f_t.half(), g_t.half(), ys_t, lx_t, ly_t)
    c_ref, _, _ = oracle.simple_loss(f_t.half().float().cpu().numpy(), g_t.half().float().cpu().numpy(), ys, lx, ly)
    assert abs(l16.item() - c_ref.mean()) < 1e-5 * c_ref.mean()


def test_reference_style_simple_class(W):
    """SimpleCTCTLoss with pre-gathered f, g and den, as the reference wires it up
    (warp_ctct/__init__.py:195-225), against the fused path."""
    N, T, U1, V = 3, 14, 6, 18
    f, g, ys, lx, ly = _case(N, T, U1, V, 17, (7, 14), (1, 5), repeat_prob=0.2)
    f_t, g_t, ys_t, lx_t, ly_t = _dev(f, g, ys, lx, ly)
    a, b = f_t.clone().requires_grad_(True), g_t.clone().requires_grad_(True)
    den = W.LogMMExp.apply(a, b.transpose(1, 2), True, True)
    idx = torch.zeros((N, T, U1), dtype=torch.long, device=DEV)
    idx[..., 1:] = ys_t.long().unsqueeze(1).expand(-1, T, -1)
    cf = a.gather(-1, idx)
    idg = torch.zeros((N, U1, 3), dtype=torch.long, device=DEV)
    idg[:, 1:, 1] = ys_t.long()
    idg[:, :U1 - 1, 2] = ys_t.long()
    cg = b.gather(-1, idg)
    cf_np, cg_np = oracle.collect_separate(f, g, ys)
    assert np.array_equal(cf.detach().cpu().numpy(), cf_np) and np.array_equal(cg.detach().cpu().numpy(), cg_np)
    costs = W.SimpleCTCTLoss.apply(cf, cg, den, ys_t, lx_t, ly_t, True, True)
    costs.sum().backward()
    c, d = f_t.clone().requires_grad_(True), g_t.clone().requires_grad_(True)
    fused = W.ctct_simple_loss(c, d, ys_t, lx_t, ly_t, reduction="none")
    fused.sum().backward()
    np.testing.assert_allclose(costs.detach().cpu().numpy(), fused.detach().cpu().numpy(), rtol=1e-5)
    assert (a.grad - c.grad).abs().max().item() < 5e-5 and (b.grad - d.grad).abs().max().item() < 5e-5


def test_sharded_simple_loss_on_one_rank_equals_the_plain_call(W):
    """Without a process group the sharded entry point is the plain loss (global batch = local batch)."""
    from warp_ctct_b200.sharded import sharded_ctct_simple_loss
    N, T, U1, V = 3, 50, 12, 128
    f, g, ys, lx, ly = _case(N, T, U1, V, 33, (25, 50), (3, 11))
    f_t, g_t, ys_t, lx_t, ly_t = _dev(f, g, ys, lx, ly)
    a, b = f_t.clone().requires_grad_(True), g_t.clone().requires_grad_(True)
    c, d = f_t.clone().requires_grad_(True), g_t.clone().requires_grad_(True)
    l1 = sharded_ctct_simple_loss(a, b, ys_t, lx_t, ly_t, reduction="mean")
    l2 = W.ctct_simple_loss(c, d, ys_t, lx_t, ly_t, reduction="mean")
    l1.backward()
    l2.backward()
    assert abs(l1.item() - l2.item()) <= 1e-6 * abs(l2.item())
    # the label patches are atomic adds (labels may repeat), so two runs agree to rounding, not bitwise
    assert (a.grad - c.grad).abs().max().item() <= 1e-6 and (b.grad - d.grad).abs().max().item() <= 1e-6
    # a shard of a larger batch: 'mean' divides by the global batch
    l3 = sharded_ctct_simple_loss(f_t, g_t, ys_t, lx_t, ly_t, global_batch=4 * N, reduction="mean")
    assert abs(l3.item() * 4 - l2.item()) <= 1e-6 * abs(l2.item())


@pytest.mark.parametrize("shape,lx,ly", [
    ((2, 1, 2, 64), [1, 1], [1, 1]),            # one frame, one label
    ((1, 3, 2, 72), [3], [1]),
    ((2, 129, 2, 64), [129, 70], [1, 1]),       # one frame past a 128-frame block
    ((1, 5, 200, 128), [5], [4]),               # far more contexts than frames, U+1 > 128 (separate GEMM kernels)
    ((3, 128, 128, 64), [128, 100, 64], [60, 50, 20]),  # exactly one tile each way
])
def test_simple_loss_tensor_core_edge_shapes(W, shape, lx, ly):
    N, T, U1, V = shape
    rng = np.random.default_rng(N * 100 + T)
    f = rng.standard_normal((N, T, V)).astype(np.float32)
    g = rng.standard_normal((N, U1, V)).astype(np.float32)
    ys = rng.integers(1, V, (N, max(U1 - 1, 0))).astype(np.int32)
    lx, ly = np.array(lx, np.int32), np.array(ly, np.int32)
    f_t, g_t = [t.requires_grad_(True) for t in _dev(f, g)]
    ys_t, lx_t, ly_t = _dev(ys, lx, ly)
    costs = W.ctct_simple_loss(f_t, g_t, ys_t, lx_t, ly_t, reduction="none")
    costs.sum().backward()
    c_ref, gf_ref, gg_ref = oracle.simple_loss(f, g, ys, lx, ly, True, dtype=np.float64)
    assert np.isfinite(c_ref).all()
    np.testing.assert_allclose(costs.detach().cpu().numpy(), c_ref, rtol=1e-5)
    np.testing.assert_allclose(f_t.grad.cpu().numpy(), gf_ref, atol=1e-4, rtol=2e-5)
    np.testing.assert_allclose(g_t.grad.cpu().numpy(), gg_ref, atol=1e-4, rtol=2e-5)


@pytest.mark.parametrize("normalized", [True, False])
def test_extension_entry_point_on_gathered_operands(W, normalized):
    """_C.ctct_loss_simple_fwd (csrc/binding.cpp:103-222) through its C-ABI counterpart
    ctct_b200_simple_gathered_forward: compose, lattice, occupancy gradient and the reductions in CUDA,
    against the oracle's restatement of the same pieces."""
    import warp_ctct._C as core
    N, T, U1, V = 4, 45, 14, 30
    f, g, ys, lx, ly = _case(N, T, U1, V, 41, (20, 45), (2, 13), repeat_prob=0.25)
    cf, cg = oracle.collect_separate(f, g, ys)
    den = oracle.log_matmul(f, g, np.float64).astype(np.float32) if normalized else None
    g3 = oracle.compose_simple(cf, cg, den)
    c64, gr64 = oracle.ctct_fwd(g3, ys, lx, ly, True, np.float64)
    gcf, gcg, gden = oracle.simple_reduce(gr64.astype(np.float32), normalized)
    cf_t, cg_t, ys_t, lx_t, ly_t = _dev(cf, cg, ys, lx, ly)
    den_t = _dev(den)[0] if normalized else torch.empty(1, device=DEV)   # the reference passes a 1-D dummy for "none"
    costs, grad_f, grad_g, grad_den = core.ctct_loss_simple_fwd(cf_t, cg_t, ys_t, den_t, lx_t, ly_t, True)
    np.testing.assert_allclose(costs.cpu().numpy(), c64, rtol=1e-5)
    assert grad_f.shape == cf_t.shape and grad_g.shape == cg_t.shape
    np.testing.assert_allclose(grad_f.cpu().numpy(), gcf, atol=1e-4, rtol=2e-5)
    np.testing.assert_allclose(grad_g.cpu().numpy(), gcg, atol=1e-4, rtol=2e-5)
    if normalized:
        np.testing.assert_allclose(grad_den.cpu().numpy(), gden, atol=1e-4, rtol=2e-5)
    else:
        assert grad_den is None
    c2, a, b, c = core.ctct_loss_simple_fwd(cf_t, cg_t, ys_t, den_t, lx_t, ly_t, False)
    assert a is None and b is None and c is None
    np.testing.assert_allclose(c2.cpu().numpy(), c64, rtol=1e-5)
    with pytest.raises(RuntimeError, match="length 3"):
        core.ctct_loss_simple_fwd(cf_t, cg_t[..., :2].contiguous(), ys_t, den_t, lx_t, ly_t, True)
    with pytest.raises(RuntimeError, match="matching the g at dim 1"):
        core.ctct_loss_simple_fwd(cf_t[..., :5].contiguous(), cg_t, ys_t, den_t, lx_t, ly_t, True)


def test_log_matmul_broadcasts_a_batch_of_one_on_the_right(W):
    """csrc/logmatmul.cu:148-167 expands rhs to the batch of the result; forward and backward."""
    from warp_ctct_b200.simple import log_matmul
    rng = np.random.default_rng(12)
    B, M, N, K = 3, 11, 7, 40
    f = rng.standard_normal((B, M, K)).astype(np.float32)
    g = rng.standard_normal((1, N, K)).astype(np.float32)
    want = oracle.log_matmul(f, np.repeat(g, B, 0), np.float64)
    f_t, g_t = _dev(f, g)
    got = log_matmul(f_t, g_t.transpose(1, 2))
    assert got.shape == (B, M, N)
    np.testing.assert_allclose(got.cpu().numpy(), want, rtol=0, atol=2e-5)
    with pytest.raises(RuntimeError, match="expanded size"):
        log_matmul(f_t[:1], _dev(np.repeat(g, B, 0))[0].transpose(1, 2))   # a batch of one on the LEFT does not broadcast
    a, b = f_t.clone().requires_grad_(True), g_t.clone().requires_grad_(True)
    go = torch.from_numpy(rng.standard_normal((B, M, N)).astype(np.float32)).to(DEV)
    W.LogMMExp.apply(a, b.transpose(1, 2), True, True).backward(go)
    c, d = f_t.clone().requires_grad_(True), g_t.clone().requires_grad_(True)
    torch.logsumexp(c[:, :, None, :] + d[:, None, :, :], -1).backward(go)
    assert b.grad.shape == d.grad.shape == (1, N, K)
    assert (a.grad - c.grad).abs().max().item() < 2e-5 and (b.grad - d.grad).abs().max().item() < 5e-5


def test_tensor_core_waits_that_give_up_fall_back_to_the_exact_kernels(W):
    """Every wait inside the tensor-core kernels is bounded.  With the bound set to zero polls each wait
    gives up before a single TMA load or MMA was issued: the kernels must raise their status word, free
    their tensor memory and return, and the exact kernels launched behind them must produce the result.
    First the forward kernel, then (forward at the normal bound, backward at zero) the backward kernels."""
    from warp_ctct_b200 import _lib
    from warp_ctct_b200.simple import log_matmul, log_matmul_tc
    lib = _lib.lib()
    rng = np.random.default_rng(77)
    B, M, N, K = 2, 150, 40, 192
    f = rng.standard_normal((B, M, K)).astype(np.float32)
    g = rng.standard_normal((B, N, K)).astype(np.float32)
    f_t, g_t = _dev(f, g)
    exact = log_matmul(f_t, g_t.transpose(1, 2))
    off = lib.ctct_b200_log_matmul_tc_flags_offset(B, M, N, K)
    try:
        _lib.check(lib.ctct_b200_debug_set_wait_limit(0), "set_wait_limit")
        den, ws = log_matmul_tc(f_t, g_t, keep_workspace=True)
        torch.cuda.synchronize()
        assert ws[off:off + 4].view(torch.int32).item() == 1, "the give-up status word must be raised"
        assert torch.equal(den, exact)          # recomputed by the exact kernel inside the same call
        # backward: planes from a healthy forward pass, every wait of the backward kernels gives up
        _lib.check(lib.ctct_b200_debug_set_wait_limit(-1), "set_wait_limit")
        a, b = f_t.clone().requires_grad_(True), g_t.clone().requires_grad_(True)
        out = W.LogMMExp.apply(a, b.transpose(1, 2), True, True)
        ws_bwd = out.grad_fn.saved_tensors[3]
        assert ws_bwd.numel() > 0 and not ws_bwd[off:off + 16].view(torch.int32).any().item()
        go = torch.from_numpy(rng.standard_normal((B, M, N)).astype(np.float32)).to(DEV)
        _lib.check(lib.ctct_b200_debug_set_wait_limit(0), "set_wait_limit")
        out.backward(go, retain_graph=True)
        torch.cuda.synchronize()
        assert ws_bwd[off:off + 4].view(torch.int32).item() == 1
    finally:
        _lib.check(lib.ctct_b200_debug_set_wait_limit(-1), "set_wait_limit")
    c, d = f_t.clone().requires_grad_(True), g_t.clone().requires_grad_(True)
    torch.logsumexp(c[:, :, None, :] + d[:, None, :, :], -1).backward(go)
    assert (a.grad - c.grad).abs().max().item() < 2e-5 and (b.grad - d.grad).abs().max().item() < 5e-5
    # and the library is healthy afterwards: the tensor-core path runs again without raising anything
    den2, ws2 = log_matmul_tc(f_t, g_t, keep_workspace=True)
    torch.cuda.synchronize()
    assert not ws2[off:off + 16].view(torch.int32).any().item()
    np.testing.assert_allclose(den2.cpu().numpy(), exact.cpu().numpy(), rtol=0, atol=2e-5)
