"""The C oracle against outputs of the reference's own ref_ctct.py (tests/golden/)."""
import numpy as np
import pytest

import oracle

KEYS = (("fw_simple", oracle.FW_SIMPLE), ("bw_simple", oracle.BW_SIMPLE),
        ("fw_shift", oracle.FW_SHIFT), ("bw_shift", oracle.BW_SHIFT))


def _cases(golden):
    return [str(n) for n in golden["names"]]


def test_collect_units_bit_exact(golden):
    for name in _cases(golden):
        lp, ys = golden[f"{name}/lp"], golden[f"{name}/ys"]
        got = oracle.collect_units(lp[None], ys[None])[0]
        assert np.array_equal(got, golden[f"{name}/units"]), name


def test_tables_match_reference(golden):
    for name in _cases(golden):
        g3, ys = golden[f"{name}/units"], golden[f"{name}/ys"]
        for key, which in KEYS:
            tab, ll = oracle.table(g3, ys, which, np.float32)
            ref = golden[f"{name}/{key}"]
            assert tab.shape == ref.shape, (name, key)
            # identical -inf pattern and identical untouched (debug-fill) cells
            assert np.array_equal(np.isneginf(tab), np.isneginf(ref)), (name, key)
            fin = np.isfinite(ref)
            np.testing.assert_allclose(tab[fin], ref[fin], rtol=2e-6, atol=2e-6, err_msg=f"{name}/{key}")
            np.testing.assert_allclose(ll, golden[f"{name}/{key}_ll"], rtol=2e-6, err_msg=f"{name}/{key}")


def test_four_variants_agree_in_double(golden):
    for name in _cases(golden):
        g3, ys = golden[f"{name}/units"], golden[f"{name}/ys"]
        lls = [oracle.table(g3, ys, which, np.float64)[1] for _, which in KEYS]
        assert max(lls) - min(lls) < 1e-9 * max(1.0, abs(lls[0])), (name, lls)


def test_demo_cost_is_the_printed_one(golden):
    # ref_ctct.py's __main__ prints cost 3.6803 for its seed-1 example
    assert round(-float(golden["demo/bw_shift_ll"]), 4) == 3.6803
    g3, ys = golden["demo/units"], golden["demo/ys"]
    assert round(-oracle.table(g3, ys, oracle.BW_SHIFT)[1], 4) == 3.6803


def test_gradient_matches_reference_autograd(golden):
    n_checked = 0
    for name in _cases(golden):
        if f"{name}/grad" not in golden:
            continue
        lp, ys, ref = golden[f"{name}/lp"], golden[f"{name}/ys"], golden[f"{name}/grad"]
        T, U1, V = lp.shape
        costs, dense = oracle.ctct_loss(lp[None], ys[None], [T], [U1 - 1])
        np.testing.assert_allclose(costs[0], -golden[f"{name}/bw_shift_ll"], rtol=2e-6)
        np.testing.assert_allclose(dense[0], ref, atol=5e-6, err_msg=name)
        n_checked += 1
    assert n_checked >= 6


def test_one_emission_per_frame(golden):
    # occupancies of all arcs leaving frame t sum to one
    for name in _cases(golden):
        lp, ys = golden[f"{name}/lp"], golden[f"{name}/ys"]
        T, U1, V = lp.shape
        g3 = oracle.collect_units(lp[None], ys[None])
        _, grads = oracle.ctct_fwd(g3, ys[None], [T], [U1 - 1], True, np.float64)
        np.testing.assert_allclose(-grads[0].sum(axis=(1, 2)), np.ones(T), atol=1e-9, err_msg=name)


@pytest.mark.parametrize("name", ["cfg1_0", "cfg1_1", "edge5", "edge6", "edge7"])
def test_finite_differences_double(golden, name):
    """Central differences of the float64 cost against the occupancy gradient, slot by slot.
    cfg1_1, edge5, edge6 and edge7 repeat adjacent labels ([4 5 2 2], [3 3 5 5], [2 2 2], [1 7 7 ...]):
    there the reference's own autograd gives NaN, so this is what pins the arcs that exist only
    when ys[u-1] != ys[u] (csrc/gather.cu:369-373)."""
    lp, ys = golden[f"{name}/lp"].astype(np.float32), golden[f"{name}/ys"]
    T, U1, V = lp.shape
    g3 = oracle.collect_units(lp[None], ys[None])
    c0, grads = oracle.ctct_fwd(g3, ys[None], [T], [U1 - 1], True, np.float64)
    rng = np.random.default_rng(0)
    eps = 1e-3  # inputs are float32, so the step must be representable
    assert np.isfinite(c0[0])
    checked = 0
    for _ in range(60):
        t, u, k = rng.integers(T), rng.integers(U1), rng.integers(3)
        if (u == 0 and k == 1) or (u == U1 - 1 and k == 2):
            continue
        gp, gm = g3.copy(), g3.copy()
        gp[0, t, u, k] += eps
        gm[0, t, u, k] -= eps
        step = float(gp[0, t, u, k]) - float(gm[0, t, u, k])
        cp, _ = oracle.ctct_fwd(gp, ys[None], [T], [U1 - 1], False, np.float64)
        cm, _ = oracle.ctct_fwd(gm, ys[None], [T], [U1 - 1], False, np.float64)
        assert abs((cp[0] - cm[0]) / step - grads[0, t, u, k]) < 1e-5, (name, t, u, k)
        checked += 1
    assert checked >= 30
    # every slot at once: the directional derivative along a random direction
    d = rng.standard_normal(g3.shape).astype(np.float32) * np.float32(2.0 ** -10)
    d[0, :, 0, 1] = 0
    d[0, :, U1 - 1, 2] = 0
    gp, gm = g3 + d, g3 - d
    cp, _ = oracle.ctct_fwd(gp, ys[None], [T], [U1 - 1], False, np.float64)
    cm, _ = oracle.ctct_fwd(gm, ys[None], [T], [U1 - 1], False, np.float64)
    want = float((grads[0] * (gp.astype(np.float64) - gm.astype(np.float64))[0]).sum())
    assert abs((cp[0] - cm[0]) - want) < 1e-6 * max(1.0, abs(want)) + 1e-7, name


def test_collect_separate_bit_exact(golden):
    cf, cg = oracle.collect_separate(golden["sep/f"], golden["sep/g"], golden["sep/ys"])
    assert np.array_equal(cf, golden["sep/cf"]) and np.array_equal(cg, golden["sep/cg"])


def test_ragged_batch_equals_per_utterance():
    rng = np.random.default_rng(3)
    N, T, U1, V = 5, 14, 6, 9
    x = rng.standard_normal((N, T, U1, V)).astype(np.float32)
    lp = x - np.log(np.exp(x).sum(-1, keepdims=True))
    ys = rng.integers(1, V, (N, U1 - 1)).astype(np.int32)
    lx = np.array([14, 9, 5, 11, 3], np.int32)
    ly = np.array([5, 3, 5, 1, 2], np.int32)
    costs, dense = oracle.ctct_loss(lp, ys, lx, ly)
    for n in range(N):
        c1, d1 = oracle.ctct_loss(lp[n:n + 1, :lx[n], :ly[n] + 1].copy(), ys[n:n + 1, :ly[n]].copy(), [lx[n]], [ly[n]])
        assert costs[n] == c1[0]
        assert np.array_equal(dense[n, :lx[n], :ly[n] + 1], d1[0])
        assert not dense[n, lx[n]:].any() and not dense[n, :, ly[n] + 1:].any()


def test_utterance_without_labels_is_the_all_blank_path():
    """ly == 0 (undefined in the reference, whose table never sets the cell its likelihood is read from): the one
    alignment emits a blank at context 0 in every frame; lx == 0 as well: the empty product, cost 0."""
    rng = np.random.default_rng(5)
    N, T, U1, V = 4, 7, 4, 6
    x = rng.standard_normal((N, T, U1, V)).astype(np.float32)
    lp = x - np.log(np.exp(x).sum(-1, keepdims=True))
    ys = rng.integers(1, V, (N, U1 - 1)).astype(np.int32)
    lx = np.array([7, 3, 0, 5], np.int32)
    ly = np.array([0, 0, 0, 2], np.int32)
    lp[1, 1, 0, 0] = -np.inf            # a forbidden blank: no alignment left
    go = np.array([1.0, 1.0, 1.0, 0.5], np.float32)
    costs, dense = oracle.ctct_loss(lp, ys, lx, ly, go)
    assert abs(costs[0] + lp[0, :7, 0, 0].sum()) < 1e-5 and np.isposinf(costs[1]) and costs[2] == 0.0
    assert np.array_equal(dense[0, :, 0, 0], -np.ones(7, np.float32)) and np.abs(dense[0]).sum() == 7.0
    assert not dense[1].any() and not dense[2].any()
    c64, g64 = oracle.ctct_fwd(oracle.collect_units(lp, ys), ys, lx, ly, True, np.float64)
    assert abs(c64[0] - costs[0]) < 1e-5 and abs(c64[3] - costs[3]) < 1e-5 and g64[0, :, 0, 0].tolist() == [-1.0] * 7


def test_round_half_matches_numpy():
    rng = np.random.default_rng(5)
    xs = np.concatenate([rng.standard_normal(2000) * 10.0 ** rng.integers(-9, 5, 2000), [0.0, 65504.0, 65519.9, 65520.0, 1e-8, -3e-8]])
    for x in xs.astype(np.float32):
        with np.errstate(over="ignore"):
            want = np.float32(np.float16(x))
        assert oracle.round_half(float(x)) == want, x


def test_simple_loss_equals_standard_loss_on_composed_joint():
    rng = np.random.default_rng(9)
    N, T, U1, V = 3, 10, 5, 12
    f = rng.standard_normal((N, T, V)).astype(np.float32)
    g = rng.standard_normal((N, U1, V)).astype(np.float32)
    ys = rng.integers(1, V, (N, U1 - 1)).astype(np.int32)
    lx, ly = np.array([10, 7, 4], np.int32), np.array([4, 2, 4], np.int32)
    joint = f[:, :, None, :] + g[:, None, :, :]
    lsm = joint - np.log(np.exp(joint.astype(np.float64)).sum(-1, keepdims=True))
    c_std, d_std = oracle.ctct_loss(lsm.astype(np.float32), ys, lx, ly)
    c_s, gf, gg = oracle.simple_loss(f, g, ys, lx, ly, normalized=True)
    np.testing.assert_allclose(c_s, c_std, rtol=1e-5)
    # chain rule through log_softmax: dJ = d - softmax * sum_v d
    d = d_std.astype(np.float64)
    dj = d - np.exp(lsm) * d.sum(-1, keepdims=True)
    np.testing.assert_allclose(gf, dj.sum(2), atol=2e-5)
    np.testing.assert_allclose(gg, dj.sum(1), atol=2e-5)
    # un-normalised: the joint itself is the log-prob
    c_u, gfu, ggu = oracle.simple_loss(f, g, ys, lx, ly, normalized=False)
    c_j, d_j = oracle.ctct_loss(joint, ys, lx, ly)
    np.testing.assert_allclose(c_u, c_j, rtol=1e-5)
    np.testing.assert_allclose(gfu, d_j.astype(np.float64).sum(2), atol=2e-5)
    np.testing.assert_allclose(ggu, d_j.astype(np.float64).sum(1), atol=2e-5)


def test_python_restatement_matches_reference_outputs(golden):
    """oracle/ref_py.py (per-cell Python loops, the reference's own style of CPU code; timed by the
    benchmark) against the reference's log-likelihoods and the C oracle's gradient."""
    import torch
    from oracle import ref_py
    for name in _cases(golden):
        lp, ys = golden[f"{name}/lp"].astype(np.float32), golden[f"{name}/ys"]
        T, U1, V = lp.shape
        if T * U1 > 400:
            continue
        cost, grad = ref_py.loss_and_gradient(lp, ys)
        want = -float(golden[f"{name}/bw_shift_ll"])
        assert abs(cost - want) <= 2e-6 * max(1.0, abs(want)), name
        _, a_ll = ref_py.forward_variables(torch.from_numpy(lp), torch.from_numpy(ys))
        assert abs(float(a_ll) - float(golden[f"{name}/fw_simple_ll"])) <= 2e-6 * max(1.0, abs(want)), name
        g3 = oracle.collect_units(lp[None], ys[None])
        _, g64 = oracle.ctct_fwd(g3, ys[None], [T], [U1 - 1], True, np.float64)
        np.testing.assert_allclose(grad.numpy(), g64[0], atol=2e-5, err_msg=name)
    # worker-process timing interface used by the benchmark (one process, tiny case)
    lp, ys = golden["cfg1_0/lp"].astype(np.float32), golden["cfg1_0/ys"]
    t = ref_py.time_utterances(lp[None], ys[None], [lp.shape[0]], [lp.shape[1] - 1], processes=1)
    assert len(t) == 1 and t[0] > 0
