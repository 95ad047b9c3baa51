"""``ot_b200_scores_noalloc``: the entry point for callers that cannot allocate.

Some users of the library run where device memory cannot be obtained when the
loss is evaluated: an inference server that has handed the whole GPU to its own
arena, or a plug-in whose execute hook is not allowed to allocate.  They cannot
create the workspace ``ot_b200_forward`` needs, so the library carries a fixed
16 MiB scratch array (4 Mi lattice cells) and this entry point uses only that.

The first test calls it through the C ABI twice in a row (the second batch is
smaller and different, so anything left in the shared scratch by the first call
would show) and compares the scores with those of ``ot_b200_forward`` on the
same inputs and with the CPU oracle, to the tolerance the other parity tests
use (1e-5 relative).  The others cover what the entry point refuses: a batch
beyond the built-in scratch, and lengths that are invalid somewhere in the
batch (NaN from the first affected utterance on, nothing written outside the
scores).

This file is named so that pytest collects it last.
"""
import ctypes

import numpy as np
import pytest
import torch

from optimized_transducer_b200 import _lib
from optimized_transducer_b200.transducer_loss import _Call
from oracle import oracle as O
from helpers import random_batch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _noalloc(dx, dt, dT, dU, n, v, scores):
    lib = _lib.load()
    stream = ctypes.c_void_p(torch.cuda.current_stream(torch.device(DEV)).cuda_stream)
    with torch.cuda.device(torch.device(DEV)):
        rc = lib.ot_b200_scores_noalloc(dx.data_ptr(), dt.data_ptr(), dT.data_ptr(), dU.data_ptr(),
                                        n, dx.size(0), v, dt.size(1), 0, scores.data_ptr(), stream)
    assert rc == _lib.OK, _lib.last_error()
    torch.cuda.synchronize()


def _scores_three_ways(seed, n, t_range, u_range, v):
    x, tg, T, U = random_batch(seed, n, t_range, u_range, v, log_softmax=True)
    dx = torch.from_numpy(x).to(DEV)
    dt = torch.from_numpy(tg).to(DEV)
    dT = torch.from_numpy(T).to(DEV)
    dU = torch.from_numpy(U).to(DEV)
    # existing entry point (caller-provided workspace)
    want = _Call(dx, dt, dT, dU, 0, True, False).forward().clone()
    # new entry point: inputs and outputs only
    got = torch.full((n,), float("nan"), dtype=torch.float32, device=DEV)
    _noalloc(dx, dt, dT, dU, n, v, got)
    oracle = O.oracle_loss(x, tg, T, U, 0, from_log_softmax=True, want_grad=False)["scores"]
    return got.cpu().numpy(), want.cpu().numpy(), oracle


def test_two_calls_in_a_row_match_the_workspace_entry_point_and_the_oracle():
    first = _scores_three_ways(901, 6, (40, 90), (10, 45), 64)
    second = _scores_three_ways(902, 3, (5, 30), (2, 12), 17)
    for got, want, oracle in (first, second):
        assert np.all(np.isfinite(got))
        assert np.max(np.abs(got - want) / np.abs(want)) <= 1e-5
        assert np.max(np.abs(got - oracle) / np.abs(oracle)) <= 1e-5


def test_batches_beyond_the_built_in_scratch_are_rejected():
    lib = _lib.load()
    one = torch.zeros(8, dtype=torch.int32, device=DEV)
    rc = lib.ot_b200_scores_noalloc(one.data_ptr(), one.data_ptr(), one.data_ptr(), one.data_ptr(),
                                    1, (4 << 20) + 1, 4, 1, 0, one.data_ptr(), None)
    assert rc == _lib.ERR_ARGUMENT
    assert "exceed the built-in scratch" in _lib.last_error()


@pytest.mark.parametrize("bad_at,bad_t,bad_u", [(2, -3, None), (0, 0, None), (1, None, -2), (1, None, 99)])
def test_an_invalid_length_poisons_the_scores_from_there_on_and_nothing_else(bad_at, bad_t, bad_u):
    """One utterance of a batch of five carries an impossible length.  Its row
    offset, and that of every utterance behind it, cannot be trusted: those
    scores are NaN, the utterances before it are computed as usual, and nothing
    is written but the scores.  The inputs and the scores sit between guard
    regions that must come back untouched."""
    n, v = 5, 11
    x, tg, T, U = random_batch(903, n, (6, 14), (2, 7), v, log_softmax=True)
    good = O.oracle_loss(x, tg, T, U, 0, from_log_softmax=True, want_grad=False)["scores"]
    Tb, Ub = T.copy(), U.copy()
    if bad_t is not None:
        Tb[bad_at] = bad_t
    if bad_u is not None:
        Ub[bad_at] = bad_u
    guard = 4096  # elements on either side of every buffer

    def guarded(a, fill):
        flat = torch.from_numpy(np.ascontiguousarray(a)).reshape(-1)
        buf = torch.full((flat.numel() + 2 * guard,), fill, dtype=flat.dtype, device=DEV)
        buf[guard:guard + flat.numel()] = flat.to(DEV)
        return buf, buf[guard:guard + flat.numel()].view(a.shape)

    bx, dx = guarded(x, 7.0)
    bt, dt = guarded(tg, 3)
    bT, dT = guarded(Tb, 5)
    bU, dU = guarded(Ub, 2)
    bs, scores = guarded(np.full(n, -1.0, np.float32), 9.0)
    before = [b.clone() for b in (bx, bt, bT, bU)]
    _noalloc(dx, dt, dT, dU, n, v, scores)
    got = scores.cpu().numpy()
    assert np.all(np.isnan(got[bad_at:]))
    if bad_at:
        assert np.max(np.abs(got[:bad_at] - good[:bad_at]) / np.abs(good[:bad_at])) <= 1e-5
    for b, was in zip((bx, bt, bT, bU), before):
        assert torch.equal(b, was)
    assert bool((bs[:guard] == 9.0).all()) and bool((bs[guard + n:] == 9.0).all())
    # the shared scratch is usable afterwards: a valid batch gives the oracle's scores
    got, _, oracle = _scores_three_ways(904, 4, (5, 12), (2, 6), 9)
    assert np.max(np.abs(got - oracle) / np.abs(oracle)) <= 1e-5
