"""The packing helpers (callers' side of the packed layout) against the numpy
restatement of the reference's recipe (reference README.md:165-177,
python/tests/test_compute_transducer_loss.py:36-56) and, for the padded entry
point, against the padded->packed->loss chain done by hand and torchaudio."""
import numpy as np
import pytest
import torch

import optimized_transducer_b200 as ot
from optimized_transducer_b200 import packing
from oracle import oracle as O
from helpers import random_batch, splits

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _lengths(seed, n, t_range, u_range):
    rng = np.random.default_rng(seed)
    T = rng.integers(t_range[0], t_range[1] + 1, n).astype(np.int32)
    U = rng.integers(u_range[0], u_range[1] + 1, n).astype(np.int32)
    return rng, T, U


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("d", [512, 130, 7])
def test_pack_joiner_input_forward_and_backward(d, dtype):
    rng, T, U = _lengths(5, 4, (3, 40), (0, 17))
    max_t, max_u1 = int(T.max()) + 2, int(U.max()) + 1 + 1  # padded larger than needed
    enc = rng.standard_normal((4, max_t, d)).astype(dtype)
    dec = rng.standard_normal((4, max_u1, d)).astype(dtype)
    want = O.pack_joiner_oracle(enc, dec, T, U)
    e = torch.from_numpy(enc).to(DEV).requires_grad_(True)
    q = torch.from_numpy(dec).to(DEV).requires_grad_(True)
    dT, dU = torch.from_numpy(T).to(DEV), torch.from_numpy(U).to(DEV)
    x = packing.pack_joiner_input(e, q, dT, dU)
    assert x.shape == want.shape
    np.testing.assert_array_equal(x.detach().cpu().numpy(), want)  # one addition: bit-exact
    g = rng.standard_normal(want.shape).astype(dtype)
    x.backward(torch.from_numpy(g).to(DEV))
    genc, gdec = O.pack_joiner_backward_oracle(g, T, U, max_t, max_u1)
    tol = 1e-12 if dtype == np.float64 else 2e-5
    np.testing.assert_allclose(e.grad.cpu().numpy(), genc, rtol=0, atol=tol)
    np.testing.assert_allclose(q.grad.cpu().numpy(), gdec, rtol=0, atol=tol * 4)


@pytest.mark.parametrize("d", [512, 320, 66])
def test_pack_by_frames_and_by_rows_give_the_same_bits(d, monkeypatch):
    """The joiner input has two kernels (by frames: the default; row by row:
    OT_B200_PACK=rows); same additions, so the same bits, on a ragged batch whose
    utterances span several chunks of the decoder block and several frame groups."""
    rng, T, U = _lengths(11, 7, (1, 90), (0, 60))
    T[0], U[0] = 1, 0      # smallest lattice
    T[3], U[3] = 90, 60    # largest: more than one chunk and more than one frame group
    max_t, max_u1 = int(T.max()), int(U.max()) + 1
    enc = torch.from_numpy(rng.standard_normal((7, max_t, d)).astype(np.float32)).to(DEV)
    dec = torch.from_numpy(rng.standard_normal((7, max_u1, d)).astype(np.float32)).to(DEV)
    dT, dU = torch.from_numpy(T).to(DEV), torch.from_numpy(U).to(DEV)
    monkeypatch.delenv("OT_B200_PACK", raising=False)
    by_frames = packing.pack_joiner_input(enc, dec, dT, dU).cpu().numpy()
    monkeypatch.setenv("OT_B200_PACK", "rows")
    by_rows = packing.pack_joiner_input(enc, dec, dT, dU).cpu().numpy()
    np.testing.assert_array_equal(by_frames, by_rows)
    np.testing.assert_array_equal(by_frames, O.pack_joiner_oracle(enc.cpu().numpy(), dec.cpu().numpy(), T, U))


@pytest.mark.parametrize("d", [500, 33])
def test_padded_round_trip(d):
    rng, T, U = _lengths(6, 3, (2, 25), (0, 9))
    max_t, max_u1 = int(T.max()), int(U.max()) + 1
    padded = rng.standard_normal((3, max_t, max_u1, d)).astype(np.float32)
    want = O.pack_padded_oracle(padded, T, U)
    p = torch.from_numpy(padded).to(DEV)
    dT, dU = torch.from_numpy(T).to(DEV), torch.from_numpy(U).to(DEV)
    packed = packing.pack_padded(p, dT, dU)
    np.testing.assert_array_equal(packed.cpu().numpy(), want)
    back = packing.unpack_to_padded(packed, dT, dU, max_t, max_u1).cpu().numpy()
    for b in range(3):
        np.testing.assert_array_equal(back[b, :T[b], :U[b] + 1], padded[b, :T[b], :U[b] + 1])
        assert np.all(back[b, T[b]:] == 0) and np.all(back[b, :, U[b] + 1:] == 0)


def test_inconsistent_lengths_do_not_fault_with_reports_off(monkeypatch):
    """OT_CHECKS=0: nothing is reported, but the kernels still do not follow lengths
    that exceed the padded tensors (max_t = 3 < T_b): no fault, NaN output."""
    monkeypatch.setenv("OT_CHECKS", "0")
    rng, T, U = _lengths(7, 2, (4, 6), (1, 2))
    enc = torch.zeros(2, 3, 8, device=DEV)
    dec = torch.zeros(2, 4, 8, device=DEV)
    rows = int(splits(T, U)[-1])
    out = packing.pack_joiner_input(enc, dec, torch.from_numpy(T).to(DEV), torch.from_numpy(U).to(DEV), rows=rows)
    torch.cuda.synchronize()
    assert out.shape == (rows, 8) and bool(torch.isnan(out).all())
    ot.check_inputs(DEV)  # nothing was recorded


@pytest.mark.parametrize("reduction", ["mean", "sum"])
def test_rnnt_loss_on_padded_logits(reduction):
    """The padded entry point equals pack-by-hand + packed loss, and torchaudio's
    rnnt_loss where that is importable (the reference's own oracle)."""
    x, tg, T, U = random_batch(8, 3, (6, 14), (2, 6), 11)
    sp = splits(T, U)
    max_t, max_u1 = int(T.max()), int(U.max()) + 1
    padded = np.zeros((3, max_t, max_u1, 11), np.float32)
    for b in range(3):
        padded[b, :T[b], :U[b] + 1] = x[sp[b]:sp[b + 1]].reshape(T[b], U[b] + 1, 11)
    p = torch.from_numpy(padded).to(DEV).requires_grad_(True)
    dt, dT, dU = (torch.from_numpy(a).to(DEV) for a in (tg, T, U))
    loss = packing.rnnt_loss(p, dt, dT, dU, blank=0, reduction=reduction)
    loss.backward()
    ref = O.oracle_loss(x.astype(np.float64), tg, T, U, 0)
    want = -ref["scores"].sum() / (3 if reduction == "mean" else 1)
    assert abs(loss.item() - want) <= 1e-5 * abs(want)
    scale = 1.0 / (3 if reduction == "mean" else 1)
    g = p.grad.cpu().numpy()
    for b in range(3):
        got = g[b, :T[b], :U[b] + 1].reshape(-1, 11)
        np.testing.assert_allclose(got, scale * ref["grad"][sp[b]:sp[b + 1]], rtol=0, atol=2e-5)
        assert np.all(g[b, T[b]:] == 0) and np.all(g[b, :, U[b] + 1:] == 0)
    try:
        import torchaudio
    except Exception:
        return
    ta = torchaudio.functional.rnnt_loss(torch.from_numpy(padded).requires_grad_(True), torch.from_numpy(tg),
                                         torch.from_numpy(T), torch.from_numpy(U), blank=0, reduction=reduction)
    assert abs(loss.item() - ta.item()) <= 1e-4 * abs(ta.item())


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
@pytest.mark.parametrize("d", [512, 66, 7])
def test_sixteen_bit_packing(d, dtype):
    """16-bit features (the loss accepts 16-bit logits, so the helpers before it do
    too): the joiner input is the float32 sum rounded once, which is what the
    reference's recipe gives in PyTorch; the backward sums in float32 and rounds
    once.  The oracle sees the 16-bit values widened to float64."""
    tdt = getattr(torch, dtype)
    rng, T, U = _lengths(12, 5, (2, 30), (0, 11))
    max_t, max_u1 = int(T.max()), int(U.max()) + 1
    enc = torch.from_numpy(rng.standard_normal((5, max_t, d)).astype(np.float32)).to(tdt)
    dec = torch.from_numpy(rng.standard_normal((5, max_u1, d)).astype(np.float32)).to(tdt)
    want = torch.from_numpy(O.pack_joiner_oracle(enc.double().numpy(), dec.double().numpy(), T, U)).to(tdt)
    e = enc.to(DEV).requires_grad_(True)
    q = dec.to(DEV).requires_grad_(True)
    dT, dU = torch.from_numpy(T).to(DEV), torch.from_numpy(U).to(DEV)
    x = packing.pack_joiner_input(e, q, dT, dU)
    assert x.dtype == tdt and torch.equal(x.detach().cpu(), want)
    g = torch.from_numpy(rng.standard_normal(tuple(want.shape)).astype(np.float32)).to(tdt)
    x.backward(g.to(DEV))
    genc, gdec = O.pack_joiner_backward_oracle(g.double().numpy(), T, U, max_t, max_u1)
    rel = 2.0 ** -8 if dtype == "bfloat16" else 2.0 ** -11   # half an ulp of the rounded sum, doubled
    for got, ref in ((e.grad, genc), (q.grad, gdec)):
        err = np.abs(got.double().cpu().numpy() - ref)
        assert np.all(err <= rel * np.abs(ref) + 1e-4), float(err.max())
    # padded <-> packed copies are exact in any type
    padded = torch.from_numpy(rng.standard_normal((5, max_t, max_u1, d)).astype(np.float32)).to(tdt).to(DEV)
    packed = packing.pack_padded(padded, dT, dU)
    assert torch.equal(packed.cpu(), torch.from_numpy(O.pack_padded_oracle(padded.float().cpu().numpy(), T, U)).to(tdt))
    back = packing.unpack_to_padded(packed, dT, dU, max_t, max_u1)
    assert torch.equal(packing.pack_padded(back, dT, dU), packed)


@pytest.mark.parametrize("case", [
    # dtype, D, N, T range, U range, extra padding of (max_t, max_u1)
    ("float32", 512, 24, (1, 40), (0, 30), (2, 1)),     # 16 pieces of 128 bytes per row
    ("float32", 520, 20, (3, 21), (0, 127), (0, 0)),    # a ragged 17th piece; U + 1 up to the kernel's 128
    ("float64", 256, 20, (2, 35), (0, 40), (1, 3)),
    ("bfloat16", 1024, 20, (2, 30), (0, 33), (3, 0)),   # pieces of 16 vectors of 4
    ("float16", 1000, 20, (1, 30), (0, 20), (0, 2)),
])
def test_backward_of_the_joiner_packing_from_one_read(case, monkeypatch):
    """Batches with enough (utterance, row piece) pairs to fill the device take both
    sums of the backward pass from ONE read of the gradient (pack_sum_slab_kernel);
    OT_B200_PACK_SUM=two keeps the two kernels that each read it.  Both against the
    float64 oracle of the reference's recipe; padding (t >= T_b, u > U_b) is zero."""
    dtype, d, n, tr, ur, (pad_t, pad_u) = case
    tdt = getattr(torch, dtype)
    rng, T, U = _lengths(31, n, tr, ur)
    T[0], U[0] = tr[0], ur[0]
    T[1], U[1] = tr[1], ur[1]
    max_t, max_u1 = int(T.max()) + pad_t, int(U.max()) + 1 + pad_u
    rows = int(splits(T, U)[-1])
    g = torch.from_numpy(rng.standard_normal((rows, d)).astype(np.float32)).to(tdt)
    genc, gdec = O.pack_joiner_backward_oracle(g.double().numpy(), T, U, max_t, max_u1)
    dT, dU = torch.from_numpy(T).to(DEV), torch.from_numpy(U).to(DEV)
    rel = {"float32": 2.0 ** -22, "float64": 2.0 ** -50, "bfloat16": 2.0 ** -8, "float16": 2.0 ** -11}[dtype]
    floor = {"float32": 5e-5, "float64": 1e-12, "bfloat16": 1e-4, "float16": 1e-4}[dtype]
    for mode in (None, "two"):
        if mode is None:
            monkeypatch.delenv("OT_B200_PACK_SUM", raising=False)
        else:
            monkeypatch.setenv("OT_B200_PACK_SUM", mode)
        e = torch.zeros(n, max_t, d, dtype=tdt, device=DEV, requires_grad=True)
        q = torch.zeros(n, max_u1, d, dtype=tdt, device=DEV, requires_grad=True)
        packing.pack_joiner_input(e, q, dT, dU).backward(g.to(DEV))
        torch.cuda.synchronize()
        for name, got, ref in (("encoder", e.grad, genc), ("decoder", q.grad, gdec)):
            got = got.double().cpu().numpy()
            err = np.abs(got - ref)
            assert np.all(err <= rel * np.abs(ref) + floor), (mode, name, float(err.max()))
            assert np.all(got[ref == 0] == 0), (mode, name)  # the padding is exactly zero
    ot.check_inputs(DEV)


def test_one_read_backward_fills_nan_when_the_lengths_do_not_fit(monkeypatch):
    """The same kernel with an utterance longer than the padded tensors: it must not
    follow the lengths; every element of both gradients is NaN and the failure is
    found by the next check."""
    monkeypatch.setenv("OT_CHECKS", "1")
    monkeypatch.delenv("OT_B200_PACK_SUM", raising=False)
    rng, T, U = _lengths(32, 24, (4, 9), (1, 4))
    max_t, max_u1, d = int(T.max()), int(U.max()) + 1, 512
    lib = packing._lib.load()
    Tbad = T.copy(); Tbad[5] = max_t + 1
    rows = int(splits(Tbad, U)[-1])
    g = torch.ones(rows, d, device=DEV)
    genc = torch.zeros(24, max_t, d, device=DEV)
    gdec = torch.zeros(24, max_u1, d, device=DEV)
    dT, dU = torch.from_numpy(Tbad).to(DEV), torch.from_numpy(U).to(DEV)
    ws = packing._workspace(24, g.device)
    rc = lib.ot_b200_pack_joiner_input_backward(
        g.data_ptr(), dT.data_ptr(), dU.data_ptr(), 24, rows, d, max_t, max_u1, packing._flags(g),
        ws.data_ptr(), genc.data_ptr(), gdec.data_ptr(), packing._stream(g))
    assert rc == 0
    torch.cuda.synchronize()
    assert bool(torch.isnan(genc).all()) and bool(torch.isnan(gdec).all())
    with pytest.raises(RuntimeError, match="do not fit"):
        ot.check_inputs(DEV, wait=False)
    ot.check_inputs(DEV)


@pytest.mark.parametrize("mode", ["1", "2"])
def test_lengths_that_do_not_fit_are_reported_and_the_output_is_nan(mode, monkeypatch):
    """An utterance longer than the padded tensor: the kernels must not follow the
    lengths.  The output is NaN (never uninitialised memory), and the failure is
    raised by the call itself (OT_CHECKS=2) or by the next call into the library
    (OT_CHECKS=1) - for rnnt_loss that is the loss right behind the packing."""
    monkeypatch.setenv("OT_CHECKS", mode)
    rng, T, U = _lengths(13, 3, (4, 9), (1, 4))
    max_t, max_u1, d = int(T.max()), int(U.max()) + 1, 8
    enc = torch.from_numpy(rng.standard_normal((3, max_t, d)).astype(np.float32)).to(DEV)
    dec = torch.from_numpy(rng.standard_normal((3, max_u1, d)).astype(np.float32)).to(DEV)
    Tbad = T.copy(); Tbad[1] = max_t + 1                    # T_b > max_t, rows still consistent
    rows = int(splits(Tbad, U)[-1])
    dT, dU = torch.from_numpy(Tbad).to(DEV), torch.from_numpy(U).to(DEV)
    if mode == "2":
        with pytest.raises(RuntimeError, match="do not fit"):
            packing.pack_joiner_input(enc, dec, dT, dU, rows=rows)
    else:
        x = packing.pack_joiner_input(enc, dec, dT, dU, rows=rows)   # no exception yet
        torch.cuda.synchronize()
        assert bool(torch.isnan(x).all())
        with pytest.raises(RuntimeError, match="do not fit"):
            ot.check_inputs(DEV, wait=False)
        # the padded entry point: the loss behind the packing finds the record
        v = 6
        padded = torch.zeros(3, max_t, max_u1, v, device=DEV)
        tg = torch.ones(3, int(U.max()), dtype=torch.int32, device=DEV)
        with pytest.raises(RuntimeError, match="do not fit"):
            loss = packing.rnnt_loss(padded, tg, dT, dU, blank=0)
            torch.cuda.synchronize()
            ot.check_inputs(DEV)
    ot.check_inputs(DEV)
