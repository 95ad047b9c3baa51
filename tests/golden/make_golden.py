"""Generates ``reference_vectors.npz``: outputs of the reference's own CPU build
(``oracle/_ref``, see ``oracle/build_ref.py``) on small seeded batches.

Run where the reference tree is present:  ``python tests/golden/make_golden.py``.
The file is committed; the tests only read it.  For every case the archive holds
the inputs (x, targets, T, U, blank and the two mode flags) and the reference's
scores, gradient, log-probs, alpha, beta and beta-side scores.  Cells the
reference leaves uninitialised (the symbol column at u == U, off-band alpha/beta
of the one-symbol-per-frame recursion) are stored as NaN.

The shapes are those of the reference's own tests (python/tests/test_cuda.py:15-21,
test_log_softmax.py:25-31, a scaled-down test_max_symbol_per_frame.py:16-22) plus
edge cases the reference never tests: U = 0, T = 1, a blank id other than 0,
targets equal to the blank, and a ragged batch.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_vectors.npz")

# name, T, U, V, blank, target range (lo, hi), allow modified
SHAPES = [
    ("ref_test_cuda", [3, 4], [2, 2], 3, 0, (1, 2), True),
    ("ref_test_log_softmax", [8, 5], [3, 4], 3, 0, (1, 2), True),
    ("ref_test_one_sym_small", [27, 53], [12, 15], 20, 0, (1, 19), True),
    ("edge_u0_t1", [1, 5, 1, 6], [0, 0, 3, 5], 7, 0, (1, 7), False),
    ("edge_u0_t1_modified", [1, 5, 4, 6], [0, 0, 3, 5], 7, 0, (1, 7), True),
    ("blank_not_zero_targets_hit_blank", [6, 9, 4], [3, 5, 2], 5, 2, (0, 5), True),
    ("ragged_medium", [37, 21, 40], [9, 5, 10], 64, 0, (1, 64), True),
    ("wide_vocab_odd", [9, 7], [4, 6], 131, 0, (1, 131), True),
]


def main():
    if O.load_ref() is None:
        raise SystemExit("oracle/_ref is missing: run `python oracle/build_ref.py` first")
    rng = np.random.default_rng(20211224)
    out = {}
    names = []
    for name, T, U, V, blank, (lo, hi), allow_mod in SHAPES:
        T = np.array(T, np.int32)
        U = np.array(U, np.int32)
        rows = int(O.row_splits(T, U)[-1])
        x = (rng.standard_normal((rows, V)) * 1.5).astype(np.float32)
        targets = rng.integers(lo, hi, (len(T), max(int(U.max()), 1))).astype(np.int32)
        if U.max() == 0:
            targets = targets[:, :0]
        for from_ls in (False, True):
            for modified in ((False, True) if allow_mod else (False,)):
                if modified and np.any(U > T - 1):
                    continue
                xi = x
                if from_ls:
                    m = x.max(1, keepdims=True)
                    xi = (x - (m + np.log(np.exp(x - m).sum(1, keepdims=True)))).astype(np.float32)
                key = f"{name}/ls{int(from_ls)}_mod{int(modified)}"
                tg = targets if targets.shape[1] else np.zeros((len(T), 0), np.int32)
                if tg.shape[1] == 0:
                    # the reference cannot take an empty targets tensor (max of an
                    # empty tensor); such batches are covered by the oracle only
                    continue
                scores, grad = O.ref_loss(xi, tg, T, U, blank, from_ls, modified)
                st = O.ref_stages(xi, tg, T, U, blank, from_ls, modified)
                lp = st["lp"].copy()
                alpha, beta = st["alpha"].copy(), st["beta"].copy()
                last_col = np.concatenate([
                    (np.arange(t * (u + 1)) % (u + 1)) == u for t, u in zip(T, U)])
                lp[last_col, 1] = np.nan
                if modified:
                    band = O.band_mask(T, U)
                    alpha[~band] = np.nan
                    beta[~band] = np.nan
                names.append(key)
                out[key + "/x"] = xi
                out[key + "/targets"] = tg
                out[key + "/T"] = T
                out[key + "/U"] = U
                out[key + "/meta"] = np.array([blank, int(from_ls), int(modified)], np.int32)
                out[key + "/scores"] = scores
                out[key + "/scores_beta"] = st["scores_beta"]
                out[key + "/grad"] = grad
                out[key + "/lp"] = lp
                out[key + "/alpha"] = alpha
                out[key + "/beta"] = beta
    out["names"] = np.array(names)
    np.savez_compressed(OUT, **out)
    print(f"wrote {OUT}: {len(names)} cases, {os.path.getsize(OUT) / 1e6:.2f} MB")


if __name__ == "__main__":
    main()
