"""GPU parity of the packed (ragged) layout: ctct_loss_packed on the valid rows only must give exactly
what the padded entry points give on the padded tensor (which the other tests hold to the CPU oracle),
and is checked against the oracle directly as well."""
import numpy as np
import pytest
import torch

import oracle
from test_gpu_logits import oracle_from_logits
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


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("from_logits", [False, True])
@pytest.mark.parametrize("shape,seed,kw", [
    ((5, 20, 9, 16), 1, dict(lx_range=(6, 20), ly_range=(1, 8), repeat_prob=0.3)),
    ((4, 33, 17, 136), 2, dict(lx_range=(17, 33), ly_range=(3, 16))),
    ((3, 64, 33, 512), 3, dict(lx_range=(40, 64), ly_range=(8, 32))),
    ((2, 12, 5, 13), 4, dict(lx_range=(6, 12), ly_range=(1, 4))),      # rows that are not whole 16-byte vectors
])
def test_packed_equals_padded_and_oracle(W, dtype, from_logits, shape, seed, kw):
    N, T, U1, V = shape
    lp, ys, lx, ly = make_case(N, T, U1, V, 1.5, seed, **kw)
    rng = np.random.default_rng(seed)
    x = (2.0 * rng.standard_normal((N, T, U1, V))).astype(np.float32) if from_logits else lp
    x_pad = torch.from_numpy(x).to(DEV).to(dtype)
    ys_t, lx_t, ly_t = _dev(ys, lx, ly)
    go = torch.from_numpy(rng.uniform(0.3, 2.0, N).astype(np.float32)).to(DEV)
    packed = W.pack_joint(x_pad, lx_t, ly_t).contiguous().requires_grad_(True)
    assert packed.shape == (int((lx.astype(np.int64) * (ly + 1)).sum()), V)
    padded = x_pad.clone().requires_grad_(True)
    fn_pad = W.ctct_loss_from_logits if from_logits else W.ctct_loss
    for red, avg in (("none", False), ("mean", True), ("sum", False)):
        packed.grad = padded.grad = None
        a = W.ctct_loss_packed(packed, ys_t, lx_t, ly_t, reduction=red, average_frames=avg, max_frames=T, from_logits=from_logits)
        b = fn_pad(padded, ys_t, lx_t, ly_t, reduction=red, average_frames=avg)
        if red == "none":
            a.backward(go)
            b.backward(go)
        else:
            a.backward()
            b.backward()
        assert torch.equal(a.detach(), b.detach()), red
        assert packed.grad.shape == packed.shape and packed.grad.dtype == dtype
        assert torch.equal(packed.grad, W.pack_joint(padded.grad, lx_t, ly_t)), red
        back = W.unpack_joint(packed.grad, lx_t, ly_t, T, U1)
        assert torch.equal(back, padded.grad)
    # against the oracle (float32 inputs only; the 16-bit roundings are covered by the padded tests)
    if dtype == torch.float32:
        packed.grad = None
        costs = W.ctct_loss_packed(packed, ys_t, lx_t, ly_t, reduction="none", from_logits=from_logits)   # max_frames read from the device
        costs.backward(go)
        if from_logits:
            c_ref, d_ref = oracle_from_logits(x, ys, lx, ly, go.cpu().numpy())
        else:
            c_ref, d_ref = oracle.ctct_loss(lp, ys, lx, ly, go.cpu().numpy())
        fin = np.isfinite(c_ref)
        np.testing.assert_allclose(costs.detach().cpu().numpy()[fin], c_ref[fin], rtol=1e-5)
        got = W.unpack_joint(packed.grad, lx_t, ly_t, T, U1).cpu().numpy()
        assert np.abs(got - np.where(fin[:, None, None, None], d_ref, 0.0)).max() < 1e-4


def test_packed_second_backward_and_no_grad(W):
    N, T, U1, V = 3, 30, 9, 72
    lp, ys, lx, ly = make_case(N, T, U1, V, 1.5, 9, lx_range=(15, 30), ly_range=(2, 8))
    ys_t, lx_t, ly_t = _dev(ys, lx, ly)
    packed = W.pack_joint(torch.from_numpy(lp).to(DEV), lx_t, ly_t).contiguous().requires_grad_(True)
    loss = W.ctct_loss_packed(packed, ys_t, lx_t, ly_t, reduction="mean", max_frames=T)
    loss.backward(retain_graph=True)
    first = packed.grad.clone()
    packed.grad = None
    loss.backward()          # no pre-cleared buffer left: cleared and patched in the backward pass
    assert torch.equal(first, packed.grad)
    with torch.no_grad():
        l0 = W.ctct_loss_packed(packed, ys_t, lx_t, ly_t, reduction="mean", max_frames=T)
    assert not l0.requires_grad and torch.equal(l0, loss.detach())


def test_packed_lengths_that_overrun_the_tensor_touch_nothing_beyond_it(W):
    """Lengths claiming more rows than the packed tensor has: every kernel that addresses packed rows
    compares against the row count it was given and skips what lies beyond, so the call returns
    normally with a finite gradient of the tensor's own shape."""
    N, T, U1, V = 3, 20, 6, 32
    lp, ys, lx, ly = make_case(N, T, U1, V, 1.0, 5, lx_range=(10, 20), ly_range=(2, 5))
    ys_t, lx_t, ly_t = _dev(ys, lx, ly)
    packed = W.pack_joint(torch.from_numpy(lp).to(DEV), lx_t, ly_t).contiguous()
    short = packed[: packed.size(0) - 37].clone().requires_grad_(True)      # the last utterance is cut off
    for from_logits in (False, True):
        short.grad = None
        loss = W.ctct_loss_packed(short, ys_t, lx_t, ly_t, reduction="sum", max_frames=T, from_logits=from_logits)
        loss.backward()
        torch.cuda.synchronize()
        assert short.grad.shape == short.shape
        assert torch.isfinite(short.grad).all()


@pytest.mark.parametrize("N", [1, 2, 31, 32, 33, 1000, 1024, 1025, 5000, 65535])
def test_packed_row_offsets_match_a_cumulative_sum(W, N):
    """ctct_b200_packed_offsets: cu[n] = sum over m < n of min(lx, T) * (min(ly, U) + 1), cu[N] = all rows; the
    batch sizes straddle the warp and block widths of its scan."""
    from warp_ctct_b200 import _lib
    rng = np.random.default_rng(N)
    T, U1 = 300, 40
    lx = rng.integers(-3, 400, N).astype(np.int32)       # also values the kernel has to clamp
    ly = rng.integers(-2, 60, N).astype(np.int32)
    lx_t, ly_t = _dev(lx, ly)
    cu = torch.full((N + 1,), -1, dtype=torch.int64, device=DEV)
    _lib.check(_lib.lib().ctct_b200_packed_offsets(lx_t.data_ptr(), ly_t.data_ptr(), N, T, U1, cu.data_ptr(),
                                                   _lib.stream_ptr(cu.device)), "packed_offsets")
    rows = np.clip(lx, 0, T).astype(np.int64) * (np.clip(ly, 0, U1 - 1).astype(np.int64) + 1)
    want = np.concatenate([[0], np.cumsum(rows)])
    assert np.array_equal(cu.cpu().numpy(), want)
