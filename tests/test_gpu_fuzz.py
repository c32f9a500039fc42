"""Seeded random small problems through the standard-loss entry points (padded log-probs, packed layout, raw
logits) against the CPU oracle: ragged and empty lengths, utterances without labels, repeated labels, labels that
collide with the blank, vocabularies whose rows are not whole vectors, all three element types."""
import numpy as np
import pytest
import torch

import oracle
from test_gpu_logits import oracle_from_logits

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = {torch.float32: 2e-4, torch.float16: 4e-3, torch.bfloat16: 3e-2}   # absolute, on gradients of magnitude <= 2


@pytest.fixture(scope="module")
def W():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import warp_ctct_b200
    from warp_ctct_b200 import _lib
    _lib.lib()
    return warp_ctct_b200


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def _case(rng):
    N, T, U1 = int(rng.integers(1, 7)), int(rng.integers(1, 48)), int(rng.integers(1, 24))
    V = int(rng.choice([2, 3, 5, 8, 13, 16, 31, 32, 64, 100, 128]))
    x = (float(rng.choice([0.5, 1.5, 4.0])) * rng.standard_normal((N, T, U1, V))).astype(np.float32)
    ys = rng.integers(0 if rng.random() < 0.2 else 1, V, (N, max(U1 - 1, 0))).astype(np.int32)
    if U1 > 2 and rng.random() < 0.5:
        for n in range(N):
            for u in range(1, U1 - 1):
                if rng.random() < 0.4:
                    ys[n, u] = ys[n, u - 1]
    lx = rng.integers(0 if rng.random() < 0.1 else 1, T + 1, N).astype(np.int32)
    ly = rng.integers(0, U1, N).astype(np.int32)
    go = rng.uniform(0.3, 2.0, N).astype(np.float32)
    dtype = [torch.float32, torch.float16, torch.bfloat16][int(rng.integers(0, 3))]
    return x, ys, lx, ly, go, dtype


@pytest.mark.parametrize("seed", [11, 12, 13, 14])
def test_random_problems_against_the_oracle(W, seed):
    rng = np.random.default_rng(seed)
    for case in range(40):
        x, ys, lx, ly, go, dtype = _case(rng)
        N, T, U1, V = x.shape
        tag = (seed, case, x.shape, str(dtype))
        m = x.max(-1, keepdims=True)
        lp = (x - m - np.log(np.exp(x - m).sum(-1, keepdims=True))).astype(np.float32)
        lp_t = _dev(lp).to(dtype)
        ys_t, lx_t, ly_t, go_t = _dev(ys), _dev(lx), _dev(ly), _dev(go)
        # padded log-probs
        costs_ref, dense_ref = oracle.ctct_loss(lp_t.float().cpu().numpy(), ys, lx, ly, go)
        ok = np.isfinite(costs_ref)
        a = lp_t.clone().requires_grad_(True)
        costs = W.ctct_loss(a, ys_t, lx_t, ly_t, reduction="none")
        costs.backward(go_t)
        got = costs.detach().cpu().numpy()
        assert (np.isfinite(got) == ok).all(), tag
        scale = max(1.0, float(np.abs(costs_ref[ok]).max())) if ok.any() else 1.0
        assert not ok.any() or np.abs(got[ok] - costs_ref[ok]).max() < 2e-4 * scale, tag
        grad = a.grad.float().cpu().numpy()
        assert np.abs(np.where(ok[:, None, None, None], grad - dense_ref, 0.0)).max() < TOL[dtype], tag
        assert not grad[~ok].any(), tag
        # the reduced loss of the same problem, when every utterance has an alignment
        if ok.all() and (lx > 0).all():
            b = lp_t.clone().requires_grad_(True)
            loss = W.ctct_loss(b, ys_t, lx_t, ly_t, reduction="mean", average_frames=True)
            loss.backward()
            want = float((costs_ref / lx).mean())
            assert abs(loss.item() - want) < 3e-4 * max(1.0, abs(want)), tag
        # packed layout: bit-identical to the padded call
        if int((lx.astype(np.int64) * (ly + 1)).sum()) > 0:
            packed = W.pack_joint(lp_t, lx_t, ly_t).contiguous().requires_grad_(True)
            costs_p = W.ctct_loss_packed(packed, ys_t, lx_t, ly_t, reduction="none", max_frames=T)
            costs_p.backward(go_t)
            assert torch.equal(costs_p.detach(), costs.detach()), tag
            assert torch.equal(packed.grad, W.pack_joint(a.grad, lx_t, ly_t)), tag
        # raw logits
        xl = _dev(x).to(dtype).requires_grad_(True)
        costs_l = W.ctct_loss_from_logits(xl, ys_t, lx_t, ly_t, reduction="none")
        costs_l.backward(go_t)
        c_ref, g_ref = oracle_from_logits(xl.detach().float().cpu().numpy(), ys, lx, ly, go)
        okl = np.isfinite(c_ref)
        got_l = costs_l.detach().cpu().numpy()
        assert (np.isfinite(got_l) == okl).all(), tag
        if okl.any():
            assert np.abs(got_l[okl] - c_ref[okl]).max() < 3e-4 * max(1.0, float(np.abs(c_ref[okl]).max())), tag
            err = np.abs(np.where(okl[:, None, None, None], xl.grad.float().cpu().numpy() - g_ref, 0.0)).max()
            assert err < TOL[dtype], tag


@pytest.mark.parametrize("seed", [21, 22])
def test_random_simple_loss_problems_against_the_oracle(W, seed):
    """The log-add joiner on random shapes: vocabularies on both sides of what the tensor-core kernels take
    (V >= 64 and a multiple of 8), with and without the denominator, against the float64 oracle."""
    rng = np.random.default_rng(seed)
    for case in range(40):
        N, T, U1 = int(rng.integers(1, 5)), int(rng.integers(1, 70)), int(rng.integers(1, 40))
        V = int(rng.choice([2, 5, 13, 32, 64, 72, 100, 128, 136, 256]))
        sigma = float(rng.choice([0.5, 1.5, 3.0]))
        f = (sigma * rng.standard_normal((N, T, V))).astype(np.float32)
        g = (sigma * rng.standard_normal((N, U1, V))).astype(np.float32)
        ys = rng.integers(1, V, (N, max(U1 - 1, 0))).astype(np.int32)
        if U1 > 2 and rng.random() < 0.5:
            for n in range(N):
                for u in range(1, U1 - 1):
                    if rng.random() < 0.4:
                        ys[n, u] = ys[n, u - 1]
        lx = rng.integers(1, T + 1, N).astype(np.int32)
        ly = np.minimum(rng.integers(0, U1, N), lx // 2).astype(np.int32)
        go = rng.uniform(0.3, 1.5, N).astype(np.float32)
        normalized = bool(rng.random() < 0.7)
        tag = (seed, case, (N, T, U1, V), normalized)
        f_t, g_t = _dev(f).requires_grad_(True), _dev(g).requires_grad_(True)
        costs = W.ctct_simple_loss(f_t, g_t, _dev(ys), _dev(lx), _dev(ly), reduction="none", normalized=normalized)
        costs.backward(_dev(go))
        c_ref, gf_ref, gg_ref = oracle.simple_loss(f, g, ys, lx, ly, normalized, go, dtype=np.float64)
        ok = np.isfinite(c_ref)
        got = costs.detach().cpu().numpy()
        assert (np.isfinite(got) == ok).all(), tag
        if ok.any():
            assert np.abs(got[ok] - c_ref[ok]).max() < 2e-5 * max(1.0, float(np.abs(c_ref[ok]).max())), tag
        okb = ok[:, None, None]
        # sums of up to T*(U+1) occupancies: 1e-4 absolute + 2e-5 relative, as in test_gpu_simple.py
        err_f = np.abs(np.where(okb, f_t.grad.cpu().numpy() - gf_ref, 0.0)) - 2e-5 * np.abs(gf_ref)
        err_g = np.abs(np.where(okb, g_t.grad.cpu().numpy() - gg_ref, 0.0)) - 2e-5 * np.abs(gg_ref)
        assert err_f.max() < 1e-4 and err_g.max() < 1e-4, tag
