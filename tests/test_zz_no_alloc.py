"""``ot_b200_scores_noalloc``: the entry point for callers that cannot allocate.

Some users of the library run where device memory cannot be obtained when the
loss is evaluated: an inference server that has handed the whole GPU to its own
arena, or a plug-in whose execute hook is not allowed to allocate.  They cannot
create the workspace ``ot_b200_forward`` needs, so the library carries a fixed
16 MiB scratch array (4 Mi lattice cells) and this entry point uses only that.

The test calls it through the C ABI twice in a row (the second batch is smaller
and different, so anything left in the shared scratch by the first call would
show) and compares the scores with those of ``ot_b200_forward`` on the same
inputs, to the tolerance the other parity tests use (1e-5 relative).

This file is named so that pytest collects it last.
"""
import ctypes

import numpy as np
import pytest
import torch

from optimized_transducer_b200 import _lib
from optimized_transducer_b200.transducer_loss import _Call
from helpers import random_batch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _scores_both_ways(seed, n, t_range, u_range, v):
    x, tg, T, U = random_batch(seed, n, t_range, u_range, v, log_softmax=True)
    dx = torch.from_numpy(x).to(DEV)
    dt = torch.from_numpy(tg).to(DEV)
    dT = torch.from_numpy(T).to(DEV)
    dU = torch.from_numpy(U).to(DEV)
    lib = _lib.load()
    # existing entry point (caller-provided workspace)
    want = _Call(dx, dt, dT, dU, 0, True, False).forward().clone()
    # new entry point: inputs and outputs only
    got = torch.full((n,), float("nan"), dtype=torch.float32, device=DEV)
    stream = ctypes.c_void_p(torch.cuda.current_stream(torch.device(DEV)).cuda_stream)
    with torch.cuda.device(torch.device(DEV)):
        rc = lib.ot_b200_scores_noalloc(dx.data_ptr(), dt.data_ptr(), dT.data_ptr(), dU.data_ptr(),
                                        n, dx.size(0), v, dt.size(1), 0, got.data_ptr(), stream)
    assert rc == _lib.OK, _lib.last_error()
    torch.cuda.synchronize()
    return got.cpu().numpy(), want.cpu().numpy()


def test_two_calls_in_a_row_match_the_workspace_entry_point():
    got1, want1 = _scores_both_ways(901, 6, (40, 90), (10, 45), 64)
    got2, want2 = _scores_both_ways(902, 3, (5, 30), (2, 12), 17)
    for got, want in ((got1, want1), (got2, want2)):
        assert np.all(np.isfinite(got))
        assert np.max(np.abs(got - want) / np.abs(want)) <= 1e-5


def test_batches_beyond_the_built_in_scratch_are_rejected():
    lib = _lib.load()
    one = torch.zeros(8, dtype=torch.int32, device=DEV)
    rc = lib.ot_b200_scores_noalloc(one.data_ptr(), one.data_ptr(), one.data_ptr(), one.data_ptr(),
                                    1, (4 << 20) + 1, 4, 1, 0, one.data_ptr(), None)
    assert rc == _lib.ERR_ARGUMENT
    assert "exceed the built-in scratch" in _lib.last_error()
