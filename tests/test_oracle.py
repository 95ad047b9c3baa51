"""Pins the CPU oracle (``oracle/``): against the committed outputs of the
reference's own CPU build, against brute-force path enumeration, and, where
``oracle/_ref`` has been built, against the reference itself at larger sizes."""
import numpy as np
import pytest

from oracle import oracle as O
from helpers import fp32_grad_floor, golden_case, golden_names, random_batch, splits


@pytest.mark.parametrize("name", golden_names())
def test_oracle_f32_matches_reference_vectors(name):
    c = golden_case(name)
    o = O.oracle_loss(c["x"], c["targets"], c["T"], c["U"], c["blank"],
                      c["from_log_softmax"], c["modified"])
    # Same algorithm, same precision, same libm: equal up to the summation
    # order of the row-wise logsumexp.
    np.testing.assert_allclose(o["scores"], c["scores"], rtol=1e-6, atol=1e-6)
    np.testing.assert_allclose(o["scores_beta"], c["scores_beta"], rtol=1e-6, atol=1e-6)
    np.testing.assert_allclose(o["grad"], c["grad"], rtol=0,
                               atol=max(2e-6, fp32_grad_floor(c["alpha"], c["beta"])))
    ok = ~np.isnan(c["lp"])
    np.testing.assert_allclose(o["lp"][ok], c["lp"][ok], rtol=0, atol=2e-6)
    for k in ("alpha", "beta"):
        ok = ~np.isnan(c[k])
        np.testing.assert_allclose(o[k][ok], c[k][ok], rtol=1e-6, atol=2e-6)
        assert np.all(np.isnan(o[k][~ok]))  # off-band cells stay at the fill value


@pytest.mark.parametrize("name", golden_names())
def test_oracle_f64_matches_reference_vectors(name):
    c = golden_case(name)
    o = O.oracle_loss(c["x"].astype(np.float64), c["targets"], c["T"], c["U"], c["blank"],
                      c["from_log_softmax"], c["modified"])
    np.testing.assert_allclose(o["scores"], c["scores"], rtol=1e-5, atol=1e-5)
    # the reference's float32 output is up to ~15 float32 roundings away from the
    # float64 result
    np.testing.assert_allclose(o["grad"], c["grad"], rtol=0,
                               atol=max(1e-5, 8 * fp32_grad_floor(c["alpha"], c["beta"])))


@pytest.mark.parametrize("modified", [False, True])
@pytest.mark.parametrize("T,U", [(1, 0), (2, 1), (4, 3), (6, 2), (5, 4), (7, 0), (3, 2)])
def test_oracle_against_path_enumeration(T, U, modified):
    if modified and U > T - 1:
        pytest.skip("no alignment exists")
    rng = np.random.default_rng(100 * T + U)
    V = 6
    x = rng.standard_normal((T * (U + 1), V))
    tg = rng.integers(1, V, (1, max(U, 1))).astype(np.int32)[:, :U]
    o = O.oracle_loss(x, tg, [T], [U], 0, False, modified)
    lp = o["lp"].reshape(T, U + 1, 2)
    want = O.brute_force_score(lp[..., 0], lp[..., 1], modified)
    assert abs(o["scores"][0] - want) < 1e-12
    assert abs(o["scores_beta"][0] - want) < 1e-12
    # d(-log P)/d logits sums to zero over each row (softmax Jacobian) and the
    # total occupancy of the final cell's blank is one.
    assert np.abs(o["grad"].sum(1)).max() < 1e-12


def test_oracle_gradient_is_the_derivative():
    """Finite differences of the float64 oracle's loss against its gradient."""
    rng = np.random.default_rng(7)
    for modified in (False, True):
        T, U = np.array([4, 3], np.int32), np.array([2, 1], np.int32)
        V = 4
        rows = int(splits(T, U)[-1])
        x = rng.standard_normal((rows, V))
        tg = rng.integers(1, V, (2, 2)).astype(np.int32)
        base = O.oracle_loss(x, tg, T, U, 0, False, modified)
        eps = 1e-6
        for (r, v) in [(0, 0), (3, 2), (rows - 1, 0), (7, 1)]:
            xp = x.copy(); xp[r, v] += eps
            xm = x.copy(); xm[r, v] -= eps
            lp_ = -O.oracle_loss(xp, tg, T, U, 0, False, modified, want_grad=False)["scores"].sum()
            lm_ = -O.oracle_loss(xm, tg, T, U, 0, False, modified, want_grad=False)["scores"].sum()
            assert abs((lp_ - lm_) / (2 * eps) - base["grad"][r, v]) < 1e-7


def test_oracle_in_place_and_empty_targets():
    x, tg, T, U = random_batch(3, 3, (2, 6), (0, 0), 5)
    assert tg.shape[1] == 0
    a = O.oracle_loss(x.copy(), tg, T, U, 0)
    xin = x.copy()
    b = O.oracle_loss(xin, tg, T, U, 0, in_place=True)
    assert b["grad"] is xin
    np.testing.assert_array_equal(a["grad"], xin)
    # with U = 0 the only path is all blanks
    sp = splits(T, U)
    for i in range(3):
        assert abs(a["scores"][i] - a["lp"][sp[i]:sp[i + 1], 0].sum()) < 1e-5


def test_log_softmax_mode_is_consistent_with_logits_mode():
    """The reference's own self-consistency test (python/tests/test_log_softmax.py:74-80):
    the loss from logits equals the loss from log_softmax(logits)."""
    x, tg, T, U = random_batch(11, 2, (5, 8), (3, 4), 3, dtype=np.float64)
    a = O.oracle_loss(x, tg, T, U, 0, False)
    m = x.max(1, keepdims=True)
    ls = x - (m + np.log(np.exp(x - m).sum(1, keepdims=True)))
    b = O.oracle_loss(ls, tg, T, U, 0, True)
    np.testing.assert_allclose(a["scores"], b["scores"], rtol=0, atol=1e-12)
    # chain rule through log_softmax: g_logits = g_ls - softmax * sum(g_ls)
    p = np.exp(ls)
    g = b["grad"] - p * b["grad"].sum(1, keepdims=True)
    np.testing.assert_allclose(a["grad"], g, rtol=0, atol=1e-12)


@pytest.mark.parametrize("modified", [False, True])
@pytest.mark.parametrize("from_ls", [False, True])
def test_oracle_against_reference_build(modified, from_ls):
    """Larger seeded batch against the reference itself (only where it was built)."""
    if O.load_ref() is None:
        pytest.skip("oracle/_ref not built on this machine")
    x, tg, T, U = random_batch(5, 3, (30, 60), (8, 20), 50, modified=modified, log_softmax=from_ls)
    o = O.oracle_loss(x, tg, T, U, 0, from_ls, modified)
    scores, grad = O.ref_loss(x, tg, T, U, 0, from_ls, modified)
    np.testing.assert_allclose(o["scores"], scores, rtol=1e-6)
    np.testing.assert_allclose(o["grad"], grad, rtol=0,
                               atol=max(2e-6, fp32_grad_floor(o["alpha"], o["beta"])))


def test_packing_oracles_follow_the_reference_recipe():
    """numpy packing oracles vs the README's torch recipe (README.md:165-177) and its autograd."""
    import torch
    rng = np.random.default_rng(3)
    T = np.array([4, 2, 5]); U = np.array([2, 0, 3]); d = 6
    enc = rng.standard_normal((3, 6, d)); dec = rng.standard_normal((3, 5, d))
    e = torch.from_numpy(enc).requires_grad_(True); q = torch.from_numpy(dec).requires_grad_(True)
    x = torch.cat([(e[i, :T[i]].unsqueeze(1) + q[i, :U[i] + 1].unsqueeze(0)).reshape(-1, d) for i in range(3)])
    np.testing.assert_array_equal(O.pack_joiner_oracle(enc, dec, T, U), x.detach().numpy())
    g = rng.standard_normal(tuple(x.shape))
    x.backward(torch.from_numpy(g))
    genc, gdec = O.pack_joiner_backward_oracle(g, T, U, 6, 5)
    np.testing.assert_allclose(genc, e.grad.numpy(), atol=1e-12)
    np.testing.assert_allclose(gdec, q.grad.numpy(), atol=1e-12)
    padded = rng.standard_normal((3, 6, 5, d))
    want = np.concatenate([padded[i, :T[i], :U[i] + 1].reshape(-1, d) for i in range(3)])
    np.testing.assert_array_equal(O.pack_padded_oracle(padded, T, U), want)
