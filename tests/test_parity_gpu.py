"""Parity of the CUDA path (through the C ABI) with the reference.

Oracles, in order of authority:
  1. ``tests/golden/reference_vectors.npz`` - outputs of the reference's own CPU
     build on small batches (committed; made by tests/golden/make_golden.py);
  2. ``oracle/`` - the C restatement of the reference's algorithm, pinned to (1)
     by tests/test_oracle.py, in float32 and float64.

Tolerances (float32 path), as the build's target states them:
  per-utterance loss      1e-5 relative
  alpha / beta, log-probs 1e-5, relative to max(1, |value|)
  gradient                1e-5 max absolute error, where float32 can express it:
                          the floor is helpers.fp32_grad_floor (two float32
                          roundings at the magnitude of the log-likelihood).
                          Beyond that magnitude the test that matters is
                          test_float32_error_is_not_worse_than_the_references.
float64 path: 1e-10 for all of the above.
"""
import ctypes
import os

import numpy as np
import pytest
import torch

import optimized_transducer_b200 as ot
from optimized_transducer_b200 import _lib, synthetic
from optimized_transducer_b200.transducer_loss import _Call
from oracle import oracle as O
from helpers import fp32_grad_floor, golden_case, golden_names, random_batch, splits

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def to_dev(x, targets, T, U):
    return (torch.from_numpy(np.ascontiguousarray(x)).to(DEV),
            torch.from_numpy(np.ascontiguousarray(targets)).to(DEV),
            torch.from_numpy(np.ascontiguousarray(T)).to(DEV),
            torch.from_numpy(np.ascontiguousarray(U)).to(DEV))


def run_cuda(x, targets, T, U, blank=0, from_ls=False, modified=False, want_grad=True):
    """scores, grad and the stage arrays of the CUDA path, as numpy."""
    dx, dt, dT, dU = to_dev(x, targets, T, U)
    st = ot.stage_outputs(dx, dt, dT, dU, blank, from_ls, modified)
    out = {k: (None if v is None else v.cpu().numpy()) for k, v in st.items()}
    if want_grad:
        dx.requires_grad_(True)
        scores, grad = ot.compute_transducer_loss(dx, dt, dT, dU, blank, from_ls, modified)
        if not from_ls:
            assert grad.data_ptr() == dx.data_ptr()  # in place, reference cuda.cu:449
        else:
            assert grad.data_ptr() != dx.data_ptr()  # reference cuda.cu:444
        out["grad"] = grad.cpu().numpy()
        np.testing.assert_array_equal(scores.cpu().numpy(), out["scores"])  # deterministic
    return out


def rel_to_one(a, b):
    return np.abs(a - b) / np.maximum(1.0, np.abs(b))


def check_against(out, ref, tol=1e-5, grad_tol=None, band=None):
    assert np.max(np.abs(out["scores"] - ref["scores"]) / np.abs(ref["scores"])) <= tol
    assert np.max(rel_to_one(out["scores_beta"], ref["scores_beta"])) <= tol
    ok = ~np.isnan(ref["lp"])
    if band is not None:
        ok &= band[:, None]
    assert np.max(rel_to_one(out["lp"][ok], ref["lp"][ok])) <= tol
    for k in ("alpha", "beta"):
        ok = ~np.isnan(ref[k])
        assert np.max(rel_to_one(out[k][ok], ref[k][ok])) <= tol, k
    if "grad" in out and ref.get("grad") is not None:
        if grad_tol is None:
            grad_tol = max(tol, fp32_grad_floor(ref["alpha"], ref["beta"]))
        assert np.max(np.abs(out["grad"] - ref["grad"])) <= grad_tol


# ---------------------------------------------------------------------------
# 1. the reference's own outputs
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("name", golden_names())
def test_reference_vectors(name):
    c = golden_case(name)
    out = run_cuda(c["x"], c["targets"], c["T"], c["U"], c["blank"], c["from_log_softmax"], c["modified"])
    band = O.band_mask(c["T"], c["U"]) if c["modified"] else None
    check_against(out, c, band=band)


# ---------------------------------------------------------------------------
# 2. seeded batches against the oracle, float32 and float64
# ---------------------------------------------------------------------------
CASES = [
    # seed, N, T range, U range, V, scale
    (21, 4, (50, 100), (10, 20), 500, 1.0),     # the CPU-runnable benchmark shape
    (22, 3, (20, 40), (31, 33), 64, 1.0),       # lattice columns straddle one warp
    (23, 2, (40, 70), (63, 66), 36, 2.0),       # two to three warps
    (24, 2, (30, 50), (150, 200), 24, 1.0),     # seven warps
    (25, 5, (1, 9), (0, 6), 10, 1.0),           # tiny and ragged, T = 1 and U = 0 present
    (26, 2, (33, 47), (5, 9), 1030, 1.0),       # more than one chunk per row, V % 4 != 0
    (27, 2, (25, 30), (5, 9), 2048, 1.0),       # several 16-byte chunks per lane
]


@pytest.mark.parametrize("modified", [False, True])
@pytest.mark.parametrize("from_ls", [False, True])
@pytest.mark.parametrize("case", CASES, ids=[str(c[0]) for c in CASES])
def test_seeded_batches_float32(case, from_ls, modified):
    seed, n, tr, ur, v, scale = case
    x, tg, T, U = random_batch(seed, n, tr, ur, v, scale, modified=modified, log_softmax=from_ls)
    if tg.shape[1] == 0:
        pytest.skip("empty targets")
    ref = O.oracle_loss(x, tg, T, U, 0, from_ls, modified)
    out = run_cuda(x, tg, T, U, 0, from_ls, modified)
    check_against(out, ref, band=O.band_mask(T, U) if modified else None)
    if not from_ls:
        assert np.max(rel_to_one(out["den"][O.band_mask(T, U)] if modified else out["den"],
                                 ref["den"][O.band_mask(T, U)] if modified else ref["den"])) <= 1e-5


@pytest.mark.parametrize("modified", [False, True])
@pytest.mark.parametrize("from_ls", [False, True])
@pytest.mark.parametrize("case", CASES[:5], ids=[str(c[0]) for c in CASES[:5]])
def test_seeded_batches_float64(case, from_ls, modified):
    seed, n, tr, ur, v, scale = case
    x, tg, T, U = random_batch(seed, n, tr, ur, v, scale, modified=modified, log_softmax=from_ls,
                               dtype=np.float64)
    if tg.shape[1] == 0:
        pytest.skip("empty targets")
    ref = O.oracle_loss(x, tg, T, U, 0, from_ls, modified)
    out = run_cuda(x, tg, T, U, 0, from_ls, modified)
    check_against(out, ref, tol=1e-10, grad_tol=1e-10, band=O.band_mask(T, U) if modified else None)


def test_float32_error_is_not_worse_than_the_references():
    """On a long lattice float32 cannot hold 1e-5: the reference's own output is
    ~1e-3 away from the float64 result.  The CUDA path must be as close to the
    float64 result as the reference's algorithm in float32 is."""
    x, tg, T, U = random_batch(31, 2, (200, 300), (40, 80), 500, 2.0)
    truth = O.oracle_loss(x.astype(np.float64), tg, T, U, 0)
    ref32 = O.oracle_loss(x, tg, T, U, 0)
    out = run_cuda(x, tg, T, U, 0)
    err_ref = np.max(np.abs(ref32["grad"] - truth["grad"]))
    err_cuda = np.max(np.abs(out["grad"] - truth["grad"]))
    assert err_cuda <= 1.5 * err_ref + 1e-6, (err_cuda, err_ref)
    assert np.max(np.abs(out["scores"] - truth["scores"]) / np.abs(truth["scores"])) <= 1e-5
    assert np.max(np.abs(out["grad"] - ref32["grad"])) <= fp32_grad_floor(ref32["alpha"], ref32["beta"])


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_seeded_sweep_of_shapes_flags_and_entry_points(seed):
    """Forty random configurations per seed: 1-10 utterances, T up to 1/3/20/80/300,
    U up to 0/1/5/40/130, twelve vocabulary sizes on both sides of the kernels' shape
    limits, any blank, targets that may equal the blank, raw or log-softmax input,
    both recursions, float32 and float64, through each entry point (the reference's
    native function, its autograd surface, the one-call entry with and without host
    lengths).  Loss: 1e-5 relative (float64: 1e-10).  Gradient against the float64
    oracle: 1e-5 where float32 can hold it, else 1.5 times the larger of the float32
    floor (helpers.fp32_grad_floor) and the error that the reference's own algorithm
    makes in float32 on the same input (in most long cases the two errors agree to
    three digits: the difference from float64 is the arithmetic's, not the kernel's)."""
    rng = np.random.default_rng(seed)
    for case in range(40):
        n = int(rng.integers(1, 11))
        tmax = int(rng.choice([1, 3, 20, 80, 300]))
        umax = int(rng.choice([0, 1, 5, 40, 130]))
        v = int(rng.choice([2, 3, 7, 37, 64, 260, 300, 500, 512, 513, 1024, 1030]))
        from_ls, modified = bool(rng.integers(0, 2)), bool(rng.integers(0, 2))
        blank = int(rng.choice([0, v - 1, int(rng.integers(0, v))]))
        dtype = np.float64 if rng.integers(0, 4) == 0 else np.float32
        api = str(rng.choice(["native", "autograd", "one call", "one call, host lengths"]))
        scale = float(rng.choice([0.5, 2.0, 8.0]))
        T = rng.integers(1, tmax + 1, n).astype(np.int32)
        U = rng.integers(0, umax + 1, n).astype(np.int32)
        if modified:
            U = np.minimum(U, T - 1).astype(np.int32)
        rows = int(splits(T, U)[-1])
        if rows * v > 20e6:
            continue
        x = (rng.standard_normal((rows, v)) * scale).astype(dtype)
        if from_ls:
            m = x.max(1, keepdims=True)
            x = (x - (m + np.log(np.exp(x - m).sum(1, keepdims=True)))).astype(dtype)
        tg = rng.integers(0, v, (n, max(int(U.max()), 0))).astype(np.int32)
        what = dict(seed=seed, case=case, T=T.tolist(), U=U.tolist(), v=v, from_ls=from_ls, modified=modified,
                    blank=blank, dtype=np.dtype(dtype).name, api=api)
        truth = O.oracle_loss(x.astype(np.float64), tg, T, U, blank, from_ls, modified)
        dx, dt, dT, dU = to_dev(x, tg, T, U)
        if api == "native":
            dx.requires_grad_(True)
            scores, grad = ot.compute_transducer_loss(dx, dt, dT, dU, blank, from_ls, modified)
            loss = -scores.double().sum().item()
        elif api == "autograd":
            dx.requires_grad_(True)
            out = ot.transducer_loss(dx, dt, dT, dU, blank, from_ls, modified, reduction="sum")
            out.backward()
            loss, grad = out.item(), dx.grad
        else:
            host = (torch.from_numpy(T), torch.from_numpy(U)) if api.endswith("host lengths") else None
            out, grad = ot.transducer_loss_and_grad(dx, dt, dT, dU, blank, from_ls, modified, reduction="sum",
                                                    lengths_on_host=host)
            loss = out.item()
        torch.cuda.synchronize()
        ot.check_inputs(DEV)
        want = -truth["scores"].sum()
        err = float(np.max(np.abs(grad.double().cpu().numpy() - truth["grad"]))) if rows else 0.0
        if dtype == np.float64:
            assert abs(loss - want) <= 1e-10 * max(1.0, abs(want)), what
            assert err <= 1e-10, (what, err)
            continue
        assert abs(loss - want) <= 1e-5 * max(1.0, abs(want)), what
        bound = max(1e-5, 1.5 * fp32_grad_floor(truth["alpha"], truth["beta"]))
        if err > bound:
            ref32 = O.oracle_loss(x, tg, T, U, blank, from_ls, modified)
            bound = max(bound, 1.5 * float(np.max(np.abs(ref32["grad"] - truth["grad"]))))
        assert err <= bound, (what, err, bound)


# ---------------------------------------------------------------------------
# 3. the Python surface (the reference's tests, re-expressed)
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("reduction", ["mean", "sum"])
@pytest.mark.parametrize("from_ls", [False, True])
@pytest.mark.parametrize("modified", [False, True])
@pytest.mark.parametrize("eager", ["0", "1"])
def test_autograd_surface(reduction, from_ls, modified, eager, monkeypatch):
    """Leaves -> cat -> (log_softmax) -> loss -> (loss * 3).backward(), as in the
    reference's python/tests/test_compute_transducer_loss.py:36-105."""
    monkeypatch.setenv("OT_EAGER_GRAD", eager)
    x, tg, T, U = random_batch(41, 2, (8, 12), (3, 6), 7, modified=modified)
    sp = splits(T, U)
    leaves = [torch.from_numpy(x[sp[i]:sp[i + 1]]).to(DEV).requires_grad_(True) for i in range(2)]
    logits = torch.cat(leaves)
    if from_ls:
        logits = logits.log_softmax(dim=-1)
    _, dt, dT, dU = to_dev(x, tg, T, U)
    loss = ot.transducer_loss(logits=logits, targets=dt, logit_lengths=dT, target_lengths=dU,
                              blank=0, reduction=reduction, from_log_softmax=from_ls,
                              one_sym_per_frame=modified)
    assert loss.dim() == 0
    (loss * 3).backward()
    ref = O.oracle_loss(x.astype(np.float64), tg, T, U, 0, False, modified)
    scale = 3.0 / (2 if reduction == "mean" else 1)
    want_loss = -ref["scores"].sum() / (2 if reduction == "mean" else 1)
    assert abs(loss.item() - want_loss) <= 1e-5 * abs(want_loss)
    for i in range(2):
        np.testing.assert_allclose(leaves[i].grad.cpu().numpy(), scale * ref["grad"][sp[i]:sp[i + 1]],
                                   rtol=0, atol=3e-5)


@pytest.mark.parametrize("from_ls", [False, True])
@pytest.mark.parametrize("modified", [False, True])
@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_per_utterance_loss_and_weighted_gradient(from_ls, modified, dtype):
    """The unreduced loss (no counterpart in the reference, which rejects
    reduction="none"): -scores of the oracle, and a gradient whose rows carry the
    upstream factor of their utterance."""
    x, tg, T, U = random_batch(44, 5, (6, 14), (2, 6), 9, modified=modified)
    x = x.astype(dtype)
    if from_ls:
        x = (x - np.log(np.exp(x.astype(np.float64)).sum(-1, keepdims=True))).astype(dtype)
    sp = splits(T, U)
    dx, dt, dT, dU = to_dev(x, tg, T, U)
    leaf = dx.clone().requires_grad_(True)
    loss = ot.transducer_loss_per_utterance(leaf * 1.0, dt, dT, dU, 0, from_ls, modified)
    assert loss.shape == (5,)
    w = torch.tensor([0.5, -2.0, 0.0, 3.0, 1.0], dtype=leaf.dtype, device=DEV)
    (loss * w).sum().backward()
    ref = O.oracle_loss(x.astype(np.float64), tg, T, U, 0, from_ls, modified)
    tol = 1e-5 if dtype == np.float32 else 1e-10
    np.testing.assert_allclose(loss.detach().cpu().numpy(), -ref["scores"], rtol=tol, atol=0)
    got = leaf.grad.cpu().numpy()
    for b in range(5):
        np.testing.assert_allclose(got[sp[b]:sp[b + 1]], w[b].item() * ref["grad"][sp[b]:sp[b + 1]],
                                   rtol=0, atol=3e-5 if dtype == np.float32 else 1e-10)


@pytest.mark.parametrize("modified", [False, True])
@pytest.mark.parametrize("from_ls", [False, True])
@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
@pytest.mark.parametrize("vocab", [500, 37])  # 8-byte vector path / scalar path
def test_sixteen_bit_logits_float32_math(vocab, dtype, from_ls, modified):
    """16-bit logits in, float32 arithmetic, gradient rounded back to 16 bits
    (no counterpart in the reference, which is float32 only).  The oracle sees
    exactly the values the kernels see: the 16-bit numbers widened to float64."""
    tdt = getattr(torch, dtype)
    x, tg, T, U = random_batch(45, 4, (9, 17), (3, 7), vocab, modified=modified)
    tx = torch.from_numpy(x)
    if from_ls:
        tx = tx.log_softmax(-1)
    x16 = tx.to(tdt)                      # what the kernels read
    xin = x16.to(torch.float64).numpy()   # the same numbers for the oracle
    _, dt, dT, dU = to_dev(x, tg, T, U)
    leaf = x16.to(DEV).requires_grad_(True)
    loss = ot.transducer_loss(leaf * 1, dt, dT, dU, 0, from_ls, modified, "sum")
    assert loss.dtype == torch.float32
    loss.backward()
    assert leaf.grad.dtype == tdt
    ref = O.oracle_loss(xin, tg, T, U, 0, from_ls, modified)
    want = -ref["scores"].sum()
    assert abs(loss.item() - want) <= 1e-5 * abs(want)
    got = leaf.grad.to(torch.float64).cpu().numpy()
    # rounding to nearest: half an ulp = 2^-9 (bfloat16) / 2^-12 (float16) relative,
    # plus the float32 error of the value that is rounded, plus float16's subnormal step
    rel = 2.0 ** -8 if dtype == "bfloat16" else 2.0 ** -11
    err = np.abs(got - ref["grad"])
    assert np.all(err <= rel * np.abs(ref["grad"]) + 2e-5), float(err.max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16", "float16"])
def test_bulk_copy_staged_logprob_kernel_equals_the_register_staged_one(dtype, monkeypatch):
    """Rows of 260..512 columns reach the log-prob stage through shared memory
    (16-row tiles fetched by bulk copies); OT_B200_LOGPROB=plain forces the
    kernel that loads into registers.  Same arithmetic in the same order: the
    outputs are bitwise equal, and both agree with the oracle.  33 tiles and a
    ragged tail, utterance boundaries inside tiles; the row count is even, which
    the 16-bit variant needs."""
    tdt = getattr(torch, dtype)
    T = np.array([37, 5, 64, 1, 29], np.int32)
    U = np.array([3, 9, 2, 7, 1], np.int32)
    rows = int((T.astype(np.int64) * (U + 1)).sum())
    assert rows % 2 == 0 and rows > 16 * 16
    rng = np.random.default_rng(46)
    x = torch.from_numpy((rng.standard_normal((rows, 500)) * 2).astype(np.float32)).to(tdt).to(DEV)
    tg = torch.from_numpy(rng.integers(1, 500, (5, 9)).astype(np.int32)).to(DEV)
    dT, dU = torch.from_numpy(T).to(DEV), torch.from_numpy(U).to(DEV)
    got = {}
    for mode in ("tma", "plain"):
        monkeypatch.setenv("OT_B200_LOGPROB", mode)
        got[mode] = ot.stage_outputs(x, tg, dT, dU, 0, False, False)
    for k in ("den", "lp", "scores"):
        assert torch.equal(got["tma"][k], got["plain"][k]), k
    st = got["tma"]
    ref = O.oracle_loss(x.to(torch.float64).cpu().numpy(), tg.cpu().numpy(), T, U, 0)
    assert np.max(np.abs(st["den"].double().cpu().numpy() - ref["den"]) / np.maximum(1, np.abs(ref["den"]))) <= 1e-6
    ok = ~np.isnan(ref["lp"])
    assert np.max(np.abs(st["lp"].double().cpu().numpy()[ok] - ref["lp"][ok])) <= 2e-5
    assert np.max(np.abs(st["scores"].double().cpu().numpy() - ref["scores"]) / np.abs(ref["scores"])) <= 1e-5


def test_module_form_and_no_grad():
    x, tg, T, U = random_batch(42, 3, (5, 9), (2, 4), 6)
    dx, dt, dT, dU = to_dev(x, tg, T, U)
    before = dx.clone()
    crit = ot.TransducerLoss(blank=0, reduction="sum")
    loss = crit(dx, dt, dT, dU, from_log_softmax=False)
    ref = O.oracle_loss(x, tg, T, U, 0)
    assert abs(loss.item() + ref["scores"].sum()) <= 1e-5 * abs(ref["scores"].sum())
    # no requires_grad: no gradient, logits untouched (reference cuda.cu:440-442)
    scores, grad = ot.compute_transducer_loss(dx, dt, dT, dU, 0, False, False)
    assert grad is None and torch.equal(dx, before)


def test_backward_twice_is_refused():
    x, tg, T, U = random_batch(43, 1, (4, 4), (2, 2), 5)
    dx, dt, dT, dU = to_dev(x, tg, T, U)
    leaf = dx.clone().requires_grad_(True)
    loss = ot.transducer_loss(leaf * 1.0, dt, dT, dU, 0, False)
    loss.backward(retain_graph=True)
    with pytest.raises(RuntimeError):
        loss.backward()


# ---------------------------------------------------------------------------
# 4. in-place safety, determinism, flags
# ---------------------------------------------------------------------------
def test_in_place_equals_out_of_place_bitwise():
    x, tg, T, U = random_batch(51, 3, (20, 30), (5, 12), 500, 2.0)
    dx, dt, dT, dU = to_dev(x, tg, T, U)
    call = _Call(dx, dt, dT, dU, 0, False, False)
    call.forward()
    separate = torch.full_like(dx, float("nan"))
    call.backward(separate)
    assert torch.equal(dx.cpu(), torch.from_numpy(x))  # input intact so far
    call.backward(dx)                                   # now over the logits
    assert torch.equal(separate, dx)
    ref = O.oracle_loss(x, tg, T, U, 0)
    assert np.max(np.abs(dx.cpu().numpy() - ref["grad"])) <= max(1e-5, fp32_grad_floor(ref["alpha"], ref["beta"]))


def test_scale_is_folded_into_the_gradient_pass():
    x, tg, T, U = random_batch(52, 2, (6, 9), (2, 5), 12)
    dx, dt, dT, dU = to_dev(x, tg, T, U)
    call = _Call(dx, dt, dT, dU, 0, False, False)
    call.forward()
    g1 = torch.empty_like(dx)
    g2 = torch.empty_like(dx)
    call.backward(g1)
    call.backward(g2, scale_tensor=torch.tensor(3.0, device=DEV), scale_host=0.25)
    torch.testing.assert_close(g2, g1 * 0.75, rtol=1e-6, atol=1e-7)


def test_share_sms_flag_changes_grids_not_results():
    """OT_B200_SHARE_SMS only sizes the one-wave grids one SM short."""
    x, tg, T, U = random_batch(53, 6, (30, 60), (8, 20), 500, 2.0)
    dx, dt, dT, dU = to_dev(x, tg, T, U)
    outs = []
    for share in (False, True):
        call = _Call(dx, dt, dT, dU, 0, False, False, share_sms=share)
        scores = call.forward().clone()
        g = torch.empty_like(dx)
        call.backward(g)
        outs.append((scores, g))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])


def test_stage_timeline(monkeypatch):
    """OT_TRACE=1: every stage reports when its first block started and its last
    block ended; the stages of one call follow one another."""
    monkeypatch.setenv("OT_TRACE", "1")
    x, tg, T, U = random_batch(54, 4, (30, 60), (8, 20), 64)
    dx, dt, dT, dU = to_dev(x, tg, T, U)
    call = _Call(dx, dt, dT, dU, 0, False, False)
    call.forward()
    call.backward(torch.empty_like(dx))
    torch.cuda.synchronize()
    t = call.stage("trace").cpu().numpy().reshape(20, 2)[:5]
    assert np.all(t[:, 0] > 0) and np.all(t[:, 1] >= t[:, 0])
    assert np.all(t[1:, 0] >= t[:-1, 0])          # prepare, logprob, lattice, coef, gradient start in order
    assert t[-1, 1] - t[0, 0] < 1e9                # within a second of each other (ns)
    monkeypatch.setenv("OT_TRACE", "0")
    call = _Call(dx, dt, dT, dU, 0, False, False)
    call.forward()
    torch.cuda.synchronize()
    assert int(call.stage("trace")[1]) == 0        # off: "last end" slots stay at their initial 0


@pytest.mark.parametrize("arith", ["linear", "log0", "log1"])
def test_all_recursion_arithmetics_stay_within_tolerance(arith, monkeypatch):
    """The reference's log domain with ex2/lg2.approx (OT_FAST_MATH=1) or
    expf/log1pf (=0) in the log-add, and the optional scaled linear domain
    (OT_LATTICE=linear, values m * 2^e).  The log domain is held against the
    float32 restatement of the reference (whose roundings it repeats), the linear
    domain against the float64 one (the float32 restatement is itself further
    from float64 than the bound allows)."""
    wide = (lambda a: a.astype(np.float64)) if arith == "linear" else (lambda a: a)
    x, tg, T, U = random_batch(53, 3, (30, 60), (10, 40), 50)
    ref = O.oracle_loss(wide(x), tg, T, U, 0)
    monkeypatch.setenv("OT_LATTICE", "linear" if arith == "linear" else "log")
    if arith != "linear":
        monkeypatch.setenv("OT_FAST_MATH", arith[-1])
    out = run_cuda(x, tg, T, U, 0)
    check_against(out, ref)
    x, tg, T, U = random_batch(31, 2, (200, 300), (40, 80), 500, 2.0)
    ref = O.oracle_loss(wide(x), tg, T, U, 0)
    out = run_cuda(x, tg, T, U, 0)
    check_against(out, ref)


@pytest.mark.parametrize("modified", [False, True])
def test_linear_arithmetic_on_log_probs_far_outside_the_float_exponent_range(modified, monkeypatch):
    """Log-softmax input whose target log-probs are -300 apiece (exp(-300) is not a
    float32, and the likelihood of an utterance is about exp(-300 U)), some targets
    at -inf (masked symbols) on cells that a path can avoid, and blanks near 0: the
    scaled linear recursion keeps an integer exponent beside each value, so alpha,
    beta and the scores must still match the float64 restatement at 1e-5, across
    several warps of columns (U up to 70)."""
    rng = np.random.default_rng(97)
    n, v = 3, 12
    T = np.array([90, 75, 80], np.int32)
    U = np.array([70, 33, 5], np.int32)
    if modified:
        U = np.minimum(U, T - 1).astype(np.int32)
    tg = rng.integers(1, v, (n, int(U.max()))).astype(np.int32)
    rows = int((T.astype(np.int64) * (U + 1)).sum())
    x = np.full((rows, v), -300.0, np.float32) + rng.standard_normal((rows, v)).astype(np.float32) * 20
    x[:, 0] = -np.abs(rng.standard_normal(rows)).astype(np.float32) * 1e-2  # blank: nearly certain
    sp = splits(T, U)
    # utterance 1: its first target symbol is impossible (-inf) in every second frame
    U1 = int(U[1]) + 1
    for t in range(1, int(T[1]), 2):
        x[sp[1] + t * U1 + 0, tg[1, 0]] = -np.inf
    ref = O.oracle_loss(x.astype(np.float64), tg, T, U, 0, True, modified)
    assert np.all(np.isfinite(ref["scores"])) and ref["scores"].min() < -5000
    monkeypatch.setenv("OT_LATTICE", "linear")
    out = run_cuda(x, tg, T, U, 0, from_ls=True, modified=modified)
    band = O.band_mask(T, U) if modified else np.ones(rows, bool)
    assert np.max(np.abs(out["scores"] - ref["scores"]) / np.abs(ref["scores"])) <= 1e-5
    assert np.max(rel_to_one(out["scores_beta"], ref["scores_beta"])) <= 1e-5
    for k in ("alpha", "beta"):
        want, got = ref[k][band], out[k][band]
        fin = np.isfinite(want)
        assert np.array_equal(np.isneginf(got), np.isneginf(want)), k   # unreachable cells: -inf in both
        assert np.max(rel_to_one(got[fin], want[fin])) <= 1e-5, k
    finite = lambda a: np.where(np.isfinite(a), a, 0.0)
    assert np.max(np.abs(out["grad"] - ref["grad"])) <= fp32_grad_floor(finite(ref["alpha"][band]),
                                                                         finite(ref["beta"][band]))


def test_wide_lattice_uses_generic_recursion():
    """More than 1024 lattice columns (the reference's CUDA path cannot run
    this: one thread per column, at most 1024, cuda.cu:197-205)."""
    for modified in (False, True):
        if modified:  # needs T >= U + 1
            x, tg, T, U = random_batch(54, 1, (1101, 1105), (1030, 1100), 4, modified=True)
        else:
            x, tg, T, U = random_batch(54, 2, (3, 6), (1030, 1100), 8)
        ref = O.oracle_loss(x, tg, T, U, 0, False, modified)
        out = run_cuda(x, tg, T, U, 0, False, modified)
        check_against(out, ref, band=O.band_mask(T, U) if modified else None)


def test_infeasible_utterance_gives_zero_gradient_rows():
    """-inf on every blank of one utterance: its likelihood is 0, log-likelihood
    -inf; the gradient rows of that utterance are zero (reference CUDA
    behaviour, kernels.cu:556-563), the other utterance is unaffected."""
    x, tg, T, U = random_batch(55, 2, (5, 7), (2, 3), 6)
    sp = splits(T, U)
    x[sp[0]:sp[1], 0] = -np.inf
    out = run_cuda(x, tg, T, U, 0)
    assert np.isneginf(out["scores"][0]) and np.isfinite(out["scores"][1])
    assert np.all(out["grad"][sp[0]:sp[1]] == 0)
    ref = O.oracle_loss(x[sp[1]:], tg[1:, :U[1]], T[1:], U[1:], 0)
    assert np.max(np.abs(out["grad"][sp[1]:] - ref["grad"])) <= 1e-5


def test_long_utterance_replica_float64_and_float32():
    """Four utterances of the long-utterance stress shape (T in [500,1000], U in
    [100,200], V=1024) in float64 against the float64 restatement at 1e-10, and the
    float32 path on the same numbers.  Lattices of 101..201 columns (4..7 warps)
    and up to 1200 steps: the skewed recursion runs with blocks shorter than 16
    steps here (its stages would not fit otherwise)."""
    w = synthetic.CONFIGS["cfg5"]
    T, U, tg = synthetic.make_lengths(w)
    T, U = T[:4].contiguous(), U[:4].contiguous()
    tg = tg[:4, :int(U.max())].contiguous()
    x64 = synthetic.make_logits(w, T, U, dtype=torch.float64)
    ref = O.oracle_loss(x64.numpy(), tg.numpy(), T.numpy(), U.numpy(), 0)
    dt, dT, dU = tg.to(DEV), T.to(DEV), U.to(DEV)
    for dtype, tol in ((torch.float64, 1e-10), (torch.float32, 1e-5)):
        dx = x64.to(DEV, dtype).requires_grad_(True)
        scores, grad = ot.compute_transducer_loss(dx, dt, dT, dU, 0, False, False)
        got = scores.double().cpu().numpy()
        assert np.max(np.abs(got - ref["scores"]) / np.abs(ref["scores"])) <= tol
        gerr = float((grad.double().cpu() - torch.from_numpy(ref["grad"])).abs().max())
        if dtype == torch.float64:
            assert gerr <= 1e-10
        else:
            # float32 at |log-likelihood| ~ 5000-7500 cannot hold 1e-5 against the
            # float64 result (nor can the reference): it must be as close to it as
            # the reference's algorithm run in float32, and within the float32
            # floor of that float32 result.
            ref32 = O.oracle_loss(x64.float().numpy(), tg.numpy(), T.numpy(), U.numpy(), 0)
            err_ref = float(np.abs(ref32["grad"].astype(np.float64) - ref["grad"]).max())
            assert gerr <= 1.5 * err_ref + 1e-6, (gerr, err_ref)
            g32 = float((grad.cpu() - torch.from_numpy(ref32["grad"])).abs().max())
            assert g32 <= fp32_grad_floor(ref32["alpha"], ref32["beta"]), g32
        del dx, grad


# ---------------------------------------------------------------------------
# 5. device-side input check (transducer-loss.cc:49-66) and its error path
# ---------------------------------------------------------------------------
def _expect_input_error(x, tg, T, U, match, modified=False):
    dx, dt, dT, dU = to_dev(x, tg, T, U)
    before = dx.clone()
    with pytest.raises(RuntimeError, match=match):
        ot.stage_outputs(dx, dt, dT, dU, 0, False, modified)
    torch.cuda.synchronize()
    assert torch.equal(dx, before)


def test_input_errors_are_reported_not_faulted():
    x, tg, T, U = random_batch(61, 3, (4, 6), (2, 3), 5)
    _expect_input_error(x[:-1], tg, T, U, "logits.size\\(0\\)")
    bad = tg.copy(); bad[0, 0] = 5
    _expect_input_error(x, bad, T, U, "targets.max\\(\\)")
    wide = np.concatenate([tg, np.ones((3, 1), np.int32)], axis=1)
    _expect_input_error(x, wide, T, U, "target_lengths.max")
    Tz = T.copy(); Tz[1] = 0
    _expect_input_error(x, tg, Tz, U, "logit length")
    # one symbol per frame with U > T - 1: the reference returns uninitialised memory
    T2 = np.array([3, 5], np.int32); U2 = np.array([3, 2], np.int32)
    x2 = np.zeros((int(splits(T2, U2)[-1]), 5), np.float32)
    _expect_input_error(x2, np.ones((2, 3), np.int32), T2, U2, "one_sym_per_frame", modified=True)


def test_deferred_check_reports_at_a_later_call_and_never_touches_the_logits(monkeypatch):
    """OT_CHECKS=1 (the default): the failing call returns a NaN loss without
    waiting for the device; the error is raised by a later call into the module
    (here: check_inputs, then the backward of a second failing loss), the logits
    are never written, and the next valid call works."""
    monkeypatch.setenv("OT_CHECKS", "1")
    x, tg, T, U = random_batch(63, 3, (4, 6), (2, 3), 5)
    bad = tg.copy(); bad[2, 0] = 77
    dx, dt, dT, dU = to_dev(x, bad, T, U)
    before = dx.clone()
    leaf = dx.clone().requires_grad_(True)
    logits = leaf * 1.0
    loss = ot.transducer_loss(logits, dt, dT, dU, 0, False)   # no exception here
    with pytest.raises(RuntimeError, match="targets.max\\(\\)"):
        ot.check_inputs(DEV)                                   # waits for the device, then reports
    assert torch.isnan(loss).item()
    ot.check_inputs(DEV)                                       # the record was consumed
    # the same failure, found by the backward of the loss that failed
    loss2 = ot.transducer_loss(leaf * 1.0, dt, dT, dU, 0, False)
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="an earlier call on this device"):
        loss2.backward()
    assert torch.equal(dx, before)
    # a valid call afterwards is not affected
    _, good, _, _ = to_dev(x, tg, T, U)
    ref = O.oracle_loss(x, tg, T, U, 0)
    ok = ot.transducer_loss(leaf * 1.0, good, dT, dU, 0, False, reduction="sum")
    ok.backward()
    assert abs(ok.item() + ref["scores"].sum()) <= 1e-5 * abs(ref["scores"].sum())
    ot.check_inputs(DEV)


def test_strict_check_raises_inside_the_call(monkeypatch):
    """OT_CHECKS=2: the reference's behaviour, the call itself raises."""
    monkeypatch.setenv("OT_CHECKS", "2")
    x, tg, T, U = random_batch(64, 2, (4, 6), (2, 3), 5)
    Tz = T.copy(); Tz[0] += 1
    dx, dt, dT, dU = to_dev(x, tg, Tz, U)
    with pytest.raises(RuntimeError, match="logits.size\\(0\\)"):
        ot.transducer_loss(dx, dt, dT, dU, 0, False)


def test_native_module_alias_and_reference_import_name():
    """``import optimized_transducer`` / ``import _optimized_transducer``, used the
    way the reference's python/tests/test_cuda.py:36-60 uses them (keyword
    arguments, leaves concatenated into the packed logits)."""
    import _optimized_transducer
    import optimized_transducer
    x, tg, T, U = random_batch(65, 2, (3, 4), (3, 3), 3)
    sp = splits(T, U)
    ref = O.oracle_loss(x, tg, T, U, 0)
    _, dt, dT, dU = to_dev(x, tg, T, U)
    leaves = [torch.from_numpy(x[sp[i]:sp[i + 1]]).to(DEV).requires_grad_(True) for i in range(2)]
    loss = optimized_transducer.transducer_loss(
        logits=torch.cat(leaves), targets=dt, logit_lengths=dT, target_lengths=dU, blank=0,
        reduction="sum", from_log_softmax=False)
    loss.backward()
    assert abs(loss.item() + ref["scores"].sum()) <= 1e-5 * abs(ref["scores"].sum())
    for i in range(2):
        assert np.max(np.abs(leaves[i].grad.cpu().numpy() - ref["grad"][sp[i]:sp[i + 1]])) <= 1e-5
    dx = torch.from_numpy(x).to(DEV).requires_grad_(True)
    scores, grad = _optimized_transducer.compute_transducer_loss(
        logits=dx, targets=dt, logit_lengths=dT, target_lengths=dU, blank=0,
        from_log_softmax=False, one_sym_per_frame=False)
    assert np.max(np.abs(scores.cpu().numpy() - ref["scores"]) / np.abs(ref["scores"])) <= 1e-5
    assert grad.data_ptr() == dx.data_ptr()
    assert np.max(np.abs(grad.detach().cpu().numpy() - ref["grad"])) <= 1e-5


def test_status_word_without_the_blocking_check(monkeypatch):
    monkeypatch.setenv("OT_CHECKS", "0")
    x, tg, T, U = random_batch(62, 2, (4, 6), (2, 3), 5)
    bad = tg.copy(); bad[1, 0] = 99
    dx, dt, dT, dU = to_dev(x, bad, T, U)
    call = _Call(dx, dt, dT, dU, 0, False, False)
    call.forward()  # no exception: the status stays on the device
    code, index = ctypes.c_int32(), ctypes.c_int32()
    rc = call.lib.ot_b200_read_input_status(call.workspace.data_ptr(), int(call.layout.total_bytes),
                                            ctypes.byref(code), ctypes.byref(index), None)
    assert rc == _lib.OK and code.value == 4 and index.value == 1


# ---------------------------------------------------------------------------
# 6. benchmark-sized inputs: properties that need no full-size oracle
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("name", ["cfg2", "cfg3", "cfg4"])
def test_full_size_configs(name):
    w = synthetic.CONFIGS[name]
    T, U, tg = synthetic.make_lengths(w)
    x = synthetic.make_logits(w, T, U, device=DEV)
    dT, dU, dt = T.to(DEV), U.to(DEV), tg.to(DEV)
    st = ot.stage_outputs(x, dt, dT, dU, 0, w.from_log_softmax, w.one_sym_per_frame)
    sa, sb = st["scores"].double(), st["scores_beta"].double()
    assert torch.isfinite(sa).all()
    assert ((sa - sb).abs() / sa.abs()).max().item() <= 1e-5  # the check of cpu.cc:795-797
    # two utterances against the oracle, on their own rows
    sp = splits(T.numpy(), U.numpy())
    leaf = x.clone().requires_grad_(True)
    scores, grad = ot.compute_transducer_loss(leaf, dt, dT, dU, 0, w.from_log_softmax, w.one_sym_per_frame)
    if not w.from_log_softmax:
        # d loss / d logits sums to zero over the vocabulary, up to the rounding
        # of beta at the magnitude of the log-likelihood (one ulp there is 2.4e-4)
        assert grad.sum(dim=1).abs().max().item() <= 1e-3
    for b in (0, w.n - 1):
        xb = x[sp[b]:sp[b + 1]].cpu().numpy()
        ref = O.oracle_loss(xb, tg[b:b + 1, :int(U[b])].numpy(), T[b:b + 1].numpy(), U[b:b + 1].numpy(), 0,
                            w.from_log_softmax, w.one_sym_per_frame)
        assert abs(scores[b].item() - ref["scores"][0]) <= 1e-5 * abs(ref["scores"][0])
        gb = grad[sp[b]:sp[b + 1]].cpu().numpy()
        assert np.max(np.abs(gb - ref["grad"])) <= max(1e-5, fp32_grad_floor(ref["alpha"], ref["beta"]))


@pytest.mark.parametrize("shape", ["cfg2", "cfg3", "one utterance straddles the cut", "bf16"])
def test_two_group_schedule_gives_the_same_bits(shape, monkeypatch):
    """A batch of >= 192 Mi lattice cells (768 MB of float logits) that is evaluated in one library call (the default
    schedule of transducer_loss) runs as two groups of utterances on three streams.
    Same kernels on the same data: scores, loss and gradient carry the bits of the
    one-stream schedule (OT_B200_PIPELINE=0).  Covered: the benchmark batches, a
    batch of two utterances whose first one reaches past the cut (the first group
    is then empty), and 16-bit rows."""
    if shape in ("cfg2", "cfg3", "bf16"):
        w = synthetic.CONFIGS["cfg3" if shape == "cfg3" else "cfg2"]
        T, U, tg = synthetic.make_lengths(w, n=64 if shape == "bf16" else None)  # 16-bit: twice the utterances
        x = synthetic.make_logits(w, T, U, device=DEV)
        if shape == "bf16":
            x = x.to(torch.bfloat16)
        modified, reduction = w.one_sym_per_frame, w.reduction
    else:
        T = torch.tensor([1000, 900], dtype=torch.int32)
        U = torch.tensor([230, 210], dtype=torch.int32)
        tg = torch.randint(1, 500, (2, 230), dtype=torch.int32, generator=torch.Generator().manual_seed(3))
        x = torch.randn(synthetic.num_rows(T, U), 500, device=DEV, generator=torch.Generator(device=DEV).manual_seed(4))
        modified, reduction = False, "mean"
    assert x.numel() >= 192 << 20
    dT, dU, dt = T.to(DEV), U.to(DEV), tg.to(DEV)
    got = {}
    for mode in ("0", "1"):
        monkeypatch.setenv("OT_B200_PIPELINE", mode)
        leaf = x.clone().requires_grad_(True)
        logits = leaf * 1
        loss = ot.transducer_loss(logits, dt, dT, dU, 0, False, modified, reduction)
        loss.backward()
        scores, _ = ot.compute_transducer_loss(x.clone(), dt, dT, dU, 0, False, modified)
        got[mode] = (loss.detach().clone(), leaf.grad.clone(), scores.clone())
        del leaf, logits, loss
    torch.cuda.synchronize()
    ot.check_inputs(DEV)
    for a, b in zip(got["0"], got["1"]):
        assert torch.equal(a, b)
    assert torch.isfinite(got["1"][0]).item()


@pytest.mark.parametrize("case", ["four utterances, own cuts", "four utterances, library cuts",
                                  "eleven utterances, own cuts", "two utterances", "bf16, odd cuts",
                                  "f16, odd row count",
                                  "one symbol per frame", "benchmark shard (4 of 32), timed size"])
def test_chained_group_schedule_gives_the_same_bits(case, monkeypatch):
    """Below the two-group size a one-call step is pipelined by up to four groups of
    utterances, each on streams of its own behind its part of stage 1
    (ot_b200_loss_and_gradient_groups).  Same kernels on the same data: loss and
    gradient carry the bits of the one-stream schedule (OT_B200_PIPELINE=0), and a
    bad length is reported as on one stream.  OT_B200_PIPELINE=always applies the
    schedule to batches below its size threshold."""
    modified, dtype, own, v = False, torch.float32, True, 40
    if case.startswith("four"):
        T, U = [23, 41, 17, 30], [7, 3, 9, 5]   # row counts 184, 164, 170, 180: cuts off the tile height
        own = "own" in case
    elif case.startswith("eleven"):
        T, U = [9, 14, 11, 30, 8, 12, 25, 7, 10, 16, 13], [3, 5, 2, 7, 1, 4, 6, 2, 3, 5, 4]
    elif case.startswith("two"):
        T, U = [40, 12], [6, 2]
    elif case.startswith("bf16"):
        T, U, dtype, v = [21, 33, 18, 27], [4, 6, 3, 5], torch.bfloat16, 500
    elif case.startswith("f16"):  # 597 rows: the last stage-1 launch cannot use whole 16-byte tiles
        T, U, dtype, v = [21, 33, 18, 27], [4, 6, 3, 6], torch.float16, 500
    elif case.startswith("one symbol"):
        T, U, modified = [23, 41, 17, 30], [7, 3, 9, 5], True
    else:
        w = synthetic.CONFIGS["cfg2"]
        Tt, Ut, tgt = synthetic.make_lengths(w)
        T, U, v = Tt[:4].tolist(), Ut[:4].tolist(), w.v
    T = torch.tensor(T, dtype=torch.int32)
    U = torch.tensor(U, dtype=torch.int32)
    gen = torch.Generator().manual_seed(11)
    tg = torch.randint(1, v, (T.numel(), int(U.max())), dtype=torch.int32, generator=gen)
    rows = synthetic.num_rows(T, U)
    x = (torch.randn(rows, v, generator=gen) * 2).to(DEV).to(dtype)
    dT, dU, dt = T.to(DEV), U.to(DEV), tg.to(DEV)
    host = (T, U) if own else None
    got = {}
    for mode in ("0", "always"):
        monkeypatch.setenv("OT_B200_PIPELINE", mode)
        for rep in range(2):  # twice: the second call reuses the workspace and the events
            buf = x.clone()
            loss, grad = ot.transducer_loss_and_grad(buf, dt, dT, dU, 0, False, modified, "sum",
                                                     lengths_on_host=host)
            got[mode, rep] = (loss.clone(), grad.clone())
    torch.cuda.synchronize()
    ot.check_inputs(DEV)
    for rep in range(2):
        assert torch.equal(got["0", 0][0], got["always", rep][0])
        assert torch.equal(got["0", 0][1], got["always", rep][1])
    assert torch.isfinite(got["always", 0][0]).item()
    # against the float64 oracle too (float32 cases; the bits are those of the
    # one-stream schedule, which the other tests hold to the tighter bounds)
    if dtype == torch.float32 and rows < 5000:
        ref = O.oracle_loss(x.cpu().numpy().astype(np.float64), tg.numpy(), T.numpy(), U.numpy(), 0, False, modified)
        want = -ref["scores"].sum()
        assert abs(got["always", 0][0].item() - want) <= 1e-5 * abs(want)
        np.testing.assert_allclose(got["always", 0][1].cpu().numpy(), ref["grad"], rtol=0,
                                   atol=max(3e-5, 2 * fp32_grad_floor(ref["alpha"], ref["beta"])))
    # a bad length under the grouped schedule: NaN loss, logits untouched, reported later
    monkeypatch.setenv("OT_B200_PIPELINE", "always")
    monkeypatch.setenv("OT_CHECKS", "1")
    bad = dT.clone()
    bad[0] += 1
    buf = x.clone()
    loss, _ = ot.transducer_loss_and_grad(buf, dt, bad, dU, 0, False, modified, "sum", lengths_on_host=host)
    assert torch.isnan(loss).item() and torch.equal(buf, x)
    with pytest.raises(RuntimeError, match="an earlier call on this device"):
        ot.check_inputs(DEV)


def test_two_host_threads_share_the_grouped_schedule(monkeypatch):
    """Two host threads, each on a CUDA stream of its own, call the one-call entry
    at the same time; both calls run as chained groups, i.e. they share the
    library's per-device streams and events (their enqueue sequences are
    serialised by a mutex, nothing else is).  Every result must carry the bits of
    the same input evaluated alone on one stream."""
    import threading
    shapes = [([23, 41, 17, 30], [7, 3, 9, 5]), ([19, 28, 35], [6, 4, 8])]
    v, reps = 64, 12
    data, want = [], []
    monkeypatch.setenv("OT_B200_PIPELINE", "0")
    for i, (T, U) in enumerate(shapes):
        T = torch.tensor(T, dtype=torch.int32)
        U = torch.tensor(U, dtype=torch.int32)
        gen = torch.Generator().manual_seed(100 + i)
        tg = torch.randint(1, v, (T.numel(), int(U.max())), dtype=torch.int32, generator=gen)
        xs = [(torch.randn(synthetic.num_rows(T, U), v, generator=gen) * 2).to(DEV) for _ in range(reps)]
        data.append((xs, tg.to(DEV), T.to(DEV), U.to(DEV), (T, U)))
        want.append([tuple(t.clone() for t in ot.transducer_loss_and_grad(x.clone(), tg.to(DEV), T.to(DEV), U.to(DEV),
                                                                         0, False, False, "sum")) for x in xs])
    torch.cuda.synchronize()
    monkeypatch.setenv("OT_B200_PIPELINE", "always")
    streams = [torch.cuda.Stream(device=DEV) for _ in shapes]
    got = [[] for _ in shapes]
    errors = []
    start = threading.Barrier(len(shapes))

    def worker(i):
        try:
            xs, tg, T, U, host = data[i]
            torch.cuda.set_device(DEV)
            start.wait()
            with torch.cuda.stream(streams[i]):
                for x in xs:
                    buf = x.clone()
                    loss, grad = ot.transducer_loss_and_grad(buf, tg, T, U, 0, False, False, "sum",
                                                             lengths_on_host=host)
                    got[i].append((loss.clone(), grad.clone()))
            streams[i].synchronize()
        except Exception as e:  # reported by the main thread
            errors.append(repr(e))

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(len(shapes))]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    torch.cuda.synchronize()
    assert not errors, errors
    ot.check_inputs(DEV)
    for i in range(len(shapes)):
        assert len(got[i]) == reps
        for (l0, g0), (l1, g1) in zip(want[i], got[i]):
            assert torch.equal(l0, l1) and torch.equal(g0, g1)


def test_group_cuts_are_validated():
    x, tg, T, U = random_batch(58, 3, (9, 14), (3, 6), 40)
    dx, dt, dT, dU = to_dev(x, tg, T, U)
    from optimized_transducer_b200.transducer_loss import _planned_call
    import ctypes
    call = _planned_call(dx, dt, dT, dU, 0, False, False)
    for cuts in ([0, 5, 5, dx.shape[0]], [1, 5, dx.shape[0]], [0, 5, dx.shape[0] + 1], [0, 1, 2, 3, 4, dx.shape[0]]):
        arr = (ctypes.c_int64 * len(cuts))(*cuts)
        with pytest.raises(RuntimeError, match="group_rows"):
            call.loss_and_gradient(dx, None, cuts=arr)
    ot.check_inputs(DEV)


def test_offsets_beyond_2_to_the_31_elements():
    """sum T*(U+1)*V > 2^31: the reference's kernels index with 32-bit offsets
    (kernels.cu:49) and cannot address this batch.  The LAST utterance is
    compared with the oracle run on its rows alone."""
    n, t, u, v = 12, 1000, 199, 1024
    T = np.full(n, t, np.int32); U = np.full(n, u, np.int32)
    T[-1], U[-1] = 611, 143
    rows = int(splits(T, U)[-1])
    assert rows * v > 2 ** 31
    g = torch.Generator(device=DEV).manual_seed(5)
    x = torch.randn(rows, v, generator=g, device=DEV)
    tg = torch.randint(1, v, (n, int(U.max())), dtype=torch.int32)
    dT, dU, dt = torch.from_numpy(T).to(DEV), torch.from_numpy(U).to(DEV), tg.to(DEV)
    sp = splits(T, U)
    xb = x[sp[-2]:].cpu().numpy()
    x.requires_grad_(True)
    scores, grad = ot.compute_transducer_loss(x, dt, dT, dU, 0, False, False)
    ref = O.oracle_loss(xb, tg[-1:, :U[-1]].numpy(), T[-1:], U[-1:], 0)
    assert abs(scores[-1].item() - ref["scores"][0]) <= 1e-5 * abs(ref["scores"][0])
    gb = grad[sp[-2]:].cpu().numpy()
    assert np.max(np.abs(gb - ref["grad"])) <= max(1e-5, fp32_grad_floor(ref["alpha"], ref["beta"]))


# ---------------------------------------------------------------------------
# 7. the sharded entry point on one rank (multi-rank logic: tests/test_sharding.py)
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("reduction", ["mean", "sum"])
@pytest.mark.parametrize("from_ls", [False, True])
@pytest.mark.parametrize("modified", [False, True])
def test_one_call_loss_and_grad_equals_the_oracle_and_the_autograd_surface(reduction, from_ls, modified):
    """transducer_loss_and_grad: (loss, gradient) of one library call, no autograd
    graph; three calls in a row reuse one workspace (different inputs each time)
    and each must match the fp64 oracle and, bit for bit, transducer_loss +
    backward on the same input."""
    _, tg, T, U = random_batch(51, 3, (9, 14), (3, 6), 40, modified=modified)
    rows = int((T.astype(np.int64) * (U + 1)).sum())
    for seed in (51, 52, 53):
        x = np.random.default_rng(seed).standard_normal((rows, 40)).astype(np.float32)
        if from_ls:
            m = x.max(1, keepdims=True)
            x = (x - (m + np.log(np.exp(x - m).sum(1, keepdims=True)))).astype(np.float32)
        dx, dt, dT, dU = to_dev(x, tg, T, U)
        leaf = dx.clone().requires_grad_(True)
        want = ot.transducer_loss(leaf * 1.0, dt, dT, dU, 0, from_ls, modified, reduction)
        want.backward()
        buf = dx.clone()
        loss, grad = ot.transducer_loss_and_grad(buf, dt, dT, dU, 0, from_ls, modified, reduction)
        assert (grad.data_ptr() == buf.data_ptr()) == (not from_ls)
        assert torch.equal(loss, want.detach())
        assert torch.equal(grad, leaf.grad)
        if from_ls:
            assert torch.equal(buf, dx)  # log-softmax input is left alone
        ref = O.oracle_loss(x.astype(np.float64), tg, T, U, 0, from_ls, modified)
        div = 3 if reduction == "mean" else 1
        want_loss = -ref["scores"].sum() / div
        assert abs(loss.item() - want_loss) <= 1e-5 * abs(want_loss)
        np.testing.assert_allclose(grad.cpu().numpy(), ref["grad"] / div, rtol=0, atol=2e-5)
    ot.check_inputs()


def test_one_call_loss_and_grad_reports_bad_lengths_like_the_autograd_surface(monkeypatch):
    monkeypatch.setenv("OT_CHECKS", "1")
    x, tg, T, U = random_batch(54, 3, (9, 14), (3, 6), 40)
    dx, dt, dT, dU = to_dev(x, tg, T, U)
    bad = dT.clone()
    bad[1] += 1  # the lengths no longer add up to the number of rows
    buf = dx.clone()
    loss, grad = ot.transducer_loss_and_grad(buf, dt, bad, dU, 0, False)
    assert torch.isnan(loss).item()
    assert torch.equal(buf, dx)  # nothing was written
    with pytest.raises(RuntimeError, match="an earlier call on this device"):
        ot.check_inputs()
    # and the cached plan still serves a good call afterwards
    loss, grad = ot.transducer_loss_and_grad(buf, dt, dT, dU, 0, False)
    assert torch.isfinite(loss).item()
    ot.check_inputs()


def test_sharded_one_call_entry_on_one_rank():
    from optimized_transducer_b200 import sharding
    ex = _emulated_ranks(1)[0]
    x, tg, T, U = random_batch(73, 3, (10, 20), (3, 8), 40)
    dx, dt, dT, dU = to_dev(x, tg, T, U)
    for reduction in ("mean", "sum"):
        a_buf, b_buf, c_buf = dx.clone(), dx.clone(), dx.clone()
        a, ga = ot.transducer_loss_and_grad(a_buf, dt, dT, dU, 0, False, reduction=reduction)
        b, gb = sharding.sharded_loss_and_grad(b_buf, dt, dT, dU, 0, False, reduction=reduction,
                                               global_batch=3, exchange=ex)
        sharding.wait_loss(b)
        c, gc = sharding.sharded_loss_and_grad(c_buf, dt, dT, dU, 0, False, reduction=reduction,
                                               global_batch=3)
        assert torch.allclose(a, b, rtol=1e-6) and torch.allclose(a, c, rtol=1e-6)
        assert torch.equal(ga, gb) and torch.equal(ga, gc)
    ex.check()


@pytest.mark.parametrize("reduction", ["mean", "sum"])
def test_sharded_loss_on_one_rank_equals_plain_loss(reduction):
    from optimized_transducer_b200 import sharding
    x, tg, T, U = random_batch(71, 3, (10, 20), (3, 8), 40)
    dx, dt, dT, dU = to_dev(x, tg, T, U)
    a_leaf = dx.clone().requires_grad_(True)
    b_leaf = dx.clone().requires_grad_(True)
    a = ot.transducer_loss(a_leaf * 1.0, dt, dT, dU, 0, False, reduction=reduction)
    b = sharding.sharded_transducer_loss(b_leaf * 1.0, dt, dT, dU, 0, False, reduction=reduction,
                                         overlap=True)
    (a * 2).backward()
    (b * 2).backward()
    sharding.wait_loss(b)
    assert torch.allclose(a, b, rtol=1e-6)
    assert torch.allclose(a_leaf.grad, b_leaf.grad, rtol=0, atol=1e-7)


# ---------------------------------------------------------------------------
# 8. the peer-memory scalar exchange, several ranks emulated on one device
#    (all publishes are enqueued before any gather: nothing ever waits here)
# ---------------------------------------------------------------------------
def _emulated_ranks(world, **kw):
    from optimized_transducer_b200.sharding import PeerExchange
    tables = [torch.zeros(PeerExchange.table_doubles(world), dtype=torch.float64, device=DEV)
              for _ in range(world)]
    return [PeerExchange(tables=tables, rank=r, **kw) for r in range(world)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_peer_exchange_sums_in_rank_order(dtype):
    ranks = _emulated_ranks(3)
    for step in range(300):  # wraps the ring
        vals = [torch.tensor(v * (step + 1), dtype=dtype, device=DEV) for v in (1.5, -2.25, 4.0)]
        for ex, v in zip(ranks, vals):
            ex.publish(v, step=step)
        outs = [ex.gather(torch.empty((), dtype=dtype, device=DEV), scale=0.5, step=step) for ex in ranks]
        if step in (0, 1, 255, 256, 299):
            want = 0.5 * ((1.5 * (step + 1) + -2.25 * (step + 1)) + 4.0 * (step + 1))
            for o in outs:
                assert o.item() == pytest.approx(want, rel=1e-6)
            assert outs[0].item() == outs[1].item() == outs[2].item()  # same order, same bits
    for ex in ranks:
        ex.check()


def test_one_call_exchange_and_the_sharded_loss_through_it():
    """ot_b200_exchange_allreduce (publish + gather on the library's own stream, one
    call) with a world of one: the slots are persistent memory, the value is
    defined after wait_loss; and the sharded loss routed through it equals the
    plain loss."""
    from optimized_transducer_b200 import sharding
    ex = _emulated_ranks(1)[0]
    for step in range(3):
        local, total = ex.slots(torch.float32)
        local.fill_(1.5 * (step + 1))
        ex.all_reduce_next(local, total, scale=2.0)
        sharding.wait_loss(total)
        assert total.item() == 3.0 * (step + 1)
    ex.check()
    x, tg, T, U = random_batch(72, 3, (10, 20), (3, 8), 40)
    dx, dt, dT, dU = to_dev(x, tg, T, U)
    a_leaf = dx.clone().requires_grad_(True)
    b_leaf = dx.clone().requires_grad_(True)
    a = ot.transducer_loss(a_leaf * 1.0, dt, dT, dU, 0, False, reduction="mean")
    b = sharding.sharded_transducer_loss(b_leaf * 1.0, dt, dT, dU, 0, False, reduction="mean",
                                         global_batch=3, overlap=True, exchange=ex)
    (a * 2).backward()
    (b * 2).backward()
    sharding.wait_loss(b)
    assert torch.allclose(a, b, rtol=1e-6)
    assert torch.allclose(a_leaf.grad, b_leaf.grad, rtol=0, atol=1e-7)
    ex.check()


def test_peer_exchange_gives_up_on_a_rank_that_never_publishes():
    """The wait is bounded: a flag nothing sets makes it run out; the kernel
    reports the missing rank, writes NaN and returns, the context stays usable."""
    ranks = _emulated_ranks(2, max_wait_s=0.002)
    ranks[0].publish(torch.tensor(1.0, device=DEV), step=0)
    out = ranks[0].gather(torch.zeros((), device=DEV), step=0)
    torch.cuda.synchronize()
    assert torch.isnan(out)
    with pytest.raises(RuntimeError, match="rank 1 did not publish"):
        ranks[0].check()
    assert torch.ones(4, device=DEV).sum().item() == 4.0


def test_peer_exchange_detects_an_overwritten_entry():
    from optimized_transducer_b200.sharding import PeerExchange
    ranks = _emulated_ranks(2)
    for ex in ranks:
        ex.publish(torch.tensor(1.0, device=DEV), step=PeerExchange.RING)  # same slot as step 0, one lap later
    out = ranks[1].gather(torch.zeros((), device=DEV), step=0)
    torch.cuda.synchronize()
    assert torch.isnan(out)
    with pytest.raises(RuntimeError, match="overwritten"):
        ranks[1].check()
