"""Shared helpers of the test-suite: golden-vector access and seeded batches."""
import os

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_vectors.npz")
_cache = {}


def golden():
    if "z" not in _cache:
        _cache["z"] = np.load(GOLDEN)
    return _cache["z"]


def golden_names():
    return [str(n) for n in golden()["names"]]


def golden_case(name):
    z = golden()
    c = {k: z[f"{name}/{k}"] for k in ("x", "targets", "T", "U", "meta", "scores", "scores_beta",
                                        "grad", "lp", "alpha", "beta")}
    c["blank"], c["from_log_softmax"], c["modified"] = (int(c["meta"][0]), bool(c["meta"][1]),
                                                         bool(c["meta"][2]))
    return c


def random_batch(seed, n, t_range, u_range, v, scale=1.0, modified=False, blank=0,
                 dtype=np.float32, log_softmax=False):
    """A seeded ragged batch: (x, targets, T, U)."""
    rng = np.random.default_rng(seed)
    T = rng.integers(t_range[0], t_range[1] + 1, n).astype(np.int32)
    U = rng.integers(u_range[0], u_range[1] + 1, n).astype(np.int32)
    if modified:
        U = np.minimum(U, T - 1).astype(np.int32)
    rows = int((T.astype(np.int64) * (U + 1)).sum())
    x = (rng.standard_normal((rows, v)) * scale).astype(dtype)
    if log_softmax:
        m = x.max(1, keepdims=True)
        x = (x - (m + np.log(np.exp(x - m).sum(1, keepdims=True)))).astype(dtype)
    lo = 1 if blank == 0 else 0
    targets = rng.integers(lo, v, (n, max(int(U.max()), 0))).astype(np.int32)
    return x, targets, T, U


def splits(T, U):
    return np.concatenate([[0], np.cumsum(T.astype(np.int64) * (U.astype(np.int64) + 1))])


EPS32 = float(np.finfo(np.float32).eps)


def fp32_grad_floor(alpha, beta):
    """Smallest gradient difference two faithful float32 implementations can be
    held to.  A gradient entry is exp(x + alpha + beta - L - den) with |alpha|,
    |beta|, |L| up to the magnitude M of the log-likelihood; each of them carries
    a rounding error of half an ulp(M) = M*eps/2 per addition, and entries reach
    1, so implementations that differ by one ulp in one row's logsumexp end up
    about 2*M*eps apart.  (The reference's own float32 output is 5-15x further
    than that from the float64 result; see test_parity_gpu.py.)"""
    m = max(float(np.nanmax(np.abs(alpha))), float(np.nanmax(np.abs(beta))), 1.0)
    return 2.0 * EPS32 * m
