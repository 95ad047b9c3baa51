"""The forward half computed from the joiner's operands (``ot_b200_forward_linear``,
a tcgen05 tensor-core kernel) against the path through materialised logits.

Oracle: ``logits = x @ W^T + b`` evaluated in float64 from the bfloat16 operands
(products of bfloat16 numbers are exact in float32; only the order of the
D-term sums differs), then the CPU oracle of the loss on those logits.
Tolerances: den and the log-probs to 1e-5 relative to max(1, |value|) plus the
float32 accumulation error of a D-term dot product (2e-5 absolute); scores to
1e-5 relative.
"""
import os

import numpy as np
import pytest
import torch

import optimized_transducer_b200 as ot
from oracle import oracle as O
from helpers import splits

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _case(seed, n, t_range, u_range, d, v, bias):
    rng = np.random.default_rng(seed)
    T = rng.integers(t_range[0], t_range[1] + 1, n).astype(np.int32)
    U = rng.integers(u_range[0], u_range[1] + 1, n).astype(np.int32)
    rows = int(splits(T, U)[-1])
    x = torch.from_numpy(rng.standard_normal((rows, d)).astype(np.float32)).to(torch.bfloat16)
    w = torch.from_numpy((rng.standard_normal((v, d)) / np.sqrt(d) * 2).astype(np.float32)).to(torch.bfloat16)
    b = torch.from_numpy(rng.standard_normal(v).astype(np.float32)) if bias else None
    tg = rng.integers(1, v, (n, int(U.max()))).astype(np.int32)
    logits = x.double() @ w.double().T
    if b is not None:
        logits = logits + b.double()
    return x, w, b, tg, T, U, logits.numpy()


@pytest.mark.parametrize("shape", [
    # seed, N, T range, U range, D, V, bias
    (1, 3, (5, 12), (2, 6), 64, 40, False),      # one K block, one column tile, a partial row tile
    (2, 4, (20, 40), (5, 12), 512, 500, True),   # the benchmark's shape of operands: 8 K blocks, 2 column tiles
    (3, 2, (30, 50), (3, 9), 200, 1030, True),   # D not a multiple of 64, five column tiles with a ragged last one
    (4, 5, (60, 90), (10, 30), 256, 300, False), # many row tiles per CTA
])
def test_scores_from_the_joiner_operands(shape):
    seed, n, tr, ur, d, v, bias = shape
    x, w, b, tg, T, U, logits = _case(seed, n, tr, ur, d, v, bias)
    ref = O.oracle_loss(logits, tg, T, U, 0)
    dx, dw = x.to(DEV), w.to(DEV)
    db = b.to(DEV) if b is not None else None
    dt, dT, dU = (torch.from_numpy(a).to(DEV) for a in (tg, T, U))
    out = ot.joiner_scores(dx, dw, db, dt, dT, dU, 0, stages=True)
    torch.cuda.synchronize()
    den = out["den"].double().cpu().numpy()
    assert np.max(np.abs(den - ref["den"]) / np.maximum(1, np.abs(ref["den"]))) <= 1e-5 + 2e-5
    ok = ~np.isnan(ref["lp"])
    lp = out["lp"].double().cpu().numpy()
    assert np.max(np.abs(lp[ok] - ref["lp"][ok]) / np.maximum(1, np.abs(ref["lp"][ok]))) <= 1e-5 + 4e-5
    s = out["scores"].double().cpu().numpy()
    assert np.max(np.abs(s - ref["scores"]) / np.abs(ref["scores"])) <= 1e-5
    # and the reduced loss equals the loss of the materialised float32 logits
    loss = ot.joiner_scores(dx, dw, db, dt, dT, dU, 0, reduction="mean")
    dense = (dx.float() @ dw.float().T) + (db if db is not None else 0)
    want = ot.transducer_loss(dense.contiguous(), dt, dT, dU, 0, False, reduction="mean")
    assert abs(loss.item() - want.item()) <= 2e-5 * abs(want.item())


def test_bad_lengths_are_reported_not_followed():
    x, w, b, tg, T, U, _ = _case(5, 3, (5, 9), (2, 4), 64, 20, False)
    Tb = T.copy(); Tb[1] += 1
    with pytest.raises(RuntimeError, match="logits.size\\(0\\)"):
        ot.joiner_scores(x.to(DEV), w.to(DEV), None, torch.from_numpy(tg).to(DEV),
                         torch.from_numpy(Tb).to(DEV), torch.from_numpy(U).to(DEV), 0)
    torch.cuda.synchronize()


# ---------------------------------------------------------------------------
# forward + backward without logits: joiner_loss
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("shape", [
    # seed, N, T range, U range, D, V, bias, reduction, upstream factor
    (11, 3, (5, 12), (2, 6), 64, 40, False, "sum", 1.0),     # one column tile, a partial row tile
    (12, 4, (20, 40), (5, 12), 512, 500, True, "mean", 3.0), # the benchmark's shape of operands
    (13, 2, (30, 50), (3, 9), 200, 1028, True, "sum", 0.5),  # five column tiles, the last one ragged
    (14, 3, (6, 12), (2, 5), 64, 36, False, "mean", 1.0),    # rows of 72 bytes, no bias: the padded gradient tile
])
def test_joiner_loss_gradients_against_the_materialised_path(shape):
    """d loss / d (joiner_in, weight, bias) of joiner_loss against autograd through
    float32 logits = x @ W^T + b and transducer_loss on them.  The library writes
    the gradient with respect to the logits in bfloat16, so the three contractions
    see it rounded to 2^-9 relative: each result is held to 1 % of its largest
    entry (measured: a few 1e-3), the loss itself to 2e-5."""
    seed, n, tr, ur, d, v, bias, reduction, factor = shape
    x, w, b, tg, T, U, _ = _case(seed, n, tr, ur, d, v, bias)
    dt, dT, dU = (torch.from_numpy(a).to(DEV) for a in (tg, T, U))
    xa = x.to(DEV).requires_grad_(True)
    wa = w.to(DEV).requires_grad_(True)
    ba = b.to(DEV).requires_grad_(True) if b is not None else None
    loss = ot.joiner_loss(xa, wa, ba, dt, dT, dU, 0, reduction=reduction)
    (loss * factor).backward()
    xr = x.to(DEV).float().requires_grad_(True)
    wr = w.to(DEV).float().requires_grad_(True)
    br = b.to(DEV).clone().requires_grad_(True) if b is not None else None
    logits = xr @ wr.T + (br if br is not None else 0)
    want = ot.transducer_loss(logits.contiguous(), dt, dT, dU, 0, False, reduction=reduction)
    (want * factor).backward()
    torch.cuda.synchronize()
    ot.check_inputs(DEV)
    assert abs(loss.item() - want.item()) <= 2e-5 * abs(want.item())
    pairs = [("joiner_in", xa.grad, xr.grad), ("weight", wa.grad, wr.grad)]
    if b is not None:
        pairs.append(("bias", ba.grad, br.grad))
    for name, got, ref in pairs:
        assert got.shape == ref.shape, name
        err = (got.float() - ref).abs().max().item()
        top = ref.abs().max().item()
        assert err <= 1e-2 * top, (name, err, top)


def test_gradient_with_respect_to_the_logits_entry_by_entry():
    """With W = identity (D = V) the logits ARE the rows of joiner_in and
    d loss / d joiner_in is the library's bfloat16 gradient tile itself: every entry
    against the float64 oracle gradient on those logits, to the rounding of the
    storage type (2^-8 relative) plus 2e-5."""
    rng = np.random.default_rng(21)
    n, v = 3, 64
    T = rng.integers(6, 14, n).astype(np.int32)
    U = rng.integers(2, 6, n).astype(np.int32)
    rows = int(splits(T, U)[-1])
    x = torch.from_numpy((rng.standard_normal((rows, v)) * 2).astype(np.float32)).to(torch.bfloat16)
    w = torch.eye(v, dtype=torch.bfloat16)
    tg = rng.integers(1, v, (n, int(U.max()))).astype(np.int32)
    ref = O.oracle_loss(x.double().numpy(), tg, T, U, 0)
    dt, dT, dU = (torch.from_numpy(a).to(DEV) for a in (tg, T, U))
    xa = x.to(DEV).requires_grad_(True)
    loss = ot.joiner_loss(xa, w.to(DEV), None, dt, dT, dU, 0, reduction="sum")
    loss.backward()
    torch.cuda.synchronize()
    want = -ref["scores"].sum()
    assert abs(loss.item() - want) <= 1e-5 * abs(want)
    g = xa.grad.double().cpu().numpy()
    assert np.all(np.abs(g - ref["grad"]) <= 2.0 ** -8 * np.abs(ref["grad"]) + 2e-5)


def test_joiner_loss_with_bad_lengths_gives_zero_gradients(monkeypatch):
    monkeypatch.setenv("OT_CHECKS", "1")
    x, w, b, tg, T, U, _ = _case(15, 3, (5, 9), (2, 4), 64, 20, False)
    Tb = T.copy(); Tb[1] += 1
    xa = x.to(DEV).requires_grad_(True)
    wa = w.to(DEV).requires_grad_(True)
    loss = ot.joiner_loss(xa, wa, None, torch.from_numpy(tg).to(DEV), torch.from_numpy(Tb).to(DEV),
                          torch.from_numpy(U).to(DEV), 0)
    assert torch.isnan(loss).item()
    with pytest.raises(RuntimeError, match="an earlier call on this device"):
        loss.backward()
    torch.cuda.synchronize()


def test_first_backward_of_a_process_may_be_a_small_batch():
    """The tensor maps are made by a driver call that needs the device's context
    current on the calling thread.  backward() runs on an autograd worker thread,
    and when the process has only handled small tensors so far that thread has made
    no runtime call that binds the context (its memory comes from the caching
    allocator): the library binds it and asks again.  Needs a fresh process."""
    import subprocess
    import sys
    code = (
        "import torch, optimized_transducer_b200 as ot\n"
        "dev = 'cuda:0'\n"
        "T = torch.tensor([2, 4, 5], dtype=torch.int32, device=dev)\n"
        "U = torch.tensor([0, 1, 0], dtype=torch.int32, device=dev)\n"
        "rows = int((T * (U + 1)).sum())\n"
        "x = torch.randn(rows, 64, device=dev).to(torch.bfloat16).requires_grad_(True)\n"
        "w = torch.randn(256, 64, device=dev).to(torch.bfloat16).requires_grad_(True)\n"
        "tg = torch.ones(3, 1, dtype=torch.int32, device=dev)\n"
        "loss = ot.joiner_loss(x, w, None, tg, T, U, 0, reduction='sum')\n"
        "loss.backward()\n"
        "torch.cuda.synchronize()\n"
        "assert torch.isfinite(x.grad.float()).all() and torch.isfinite(w.grad.float()).all()\n"
        "print('ok', float(loss))\n")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", code], cwd=root, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and r.stdout.startswith("ok"), (r.stdout[-300:], r.stderr[-600:])
