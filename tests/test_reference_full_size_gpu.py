"""The CUDA path against the reference's OWN build at benchmark size.

``oracle/_ref`` holds the reference's unmodified CPU implementation
(ComputeTransducerLossCpu, optimized_transducer/csrc/cpu.cc:754-827 of the
reference) compiled from its sources, plus a shim over its file-static stages.
Here it runs on the WHOLE batches of the benchmark configurations (and on the
four-utterance replica of the long-utterance one), and every utterance's score,
every alpha/beta cell and the complete gradient of the CUDA path are compared
with it, for the three arithmetics of the recursions: the reference's own log
domain with the hardware ex2/lg2 log-add ("log1": OT_FAST_MATH=1, the default
for raw logits) and with expf/log1pf ("log0": OT_FAST_MATH=0, the default for
log-softmax input), and the optional scaled linear domain ("linear":
OT_LATTICE=linear, values carried as m * 2^e).

What float32 can hold.  The score and alpha/beta tolerances are the target's:
1e-5 relative.  The gradient target, 1e-5 absolute, is met where the
log-likelihood is small (the tiny case below).  On the benchmark batches a
gradient entry is exp(x + alpha + beta - L - den) with |alpha|, |beta|, |L| in the
thousands, where one float32 rounding is 1.2e-4 to 4.9e-4: the reference's own
output is then 1e-3 and more away from the float64 result.

* In the log domain the CUDA path repeats the reference's roundings step by
  step, so it stays CLOSER to the reference than the reference is to the
  float64 result: the bounds asserted are the differences measured on B200
  with a factor 1.5 of headroom, each also required to stay below the
  reference's own distance from float64.  (For log-softmax input the exact
  log-add reproduces the reference almost to the bit, 2.5e-5 against 4.9e-4
  with the hardware approximations.)
* The linear arithmetic rounds relative to the value, not at ulp(|alpha|): its
  alpha/beta sit within one float32 rounding of the float64 recursion.  Its
  distance from the reference is therefore the reference's own distance from
  float64 (triangle inequality; asserted with 25 % slack), and its distance
  from float64 must be at most HALF the reference's.

The test prints one table row per configuration; with OT_PARITY_REPORT=<path> it
also writes them as JSON.
"""
import json
import os

import numpy as np
import pytest
import torch

import optimized_transducer_b200 as ot
from optimized_transducer_b200 import synthetic
from oracle import oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

# max |gradient(CUDA) - gradient(reference build)| allowed with the log-domain
# recursions, per configuration and log-add variant ("log1": ex2/lg2.approx,
# "log0": expf/log1pf)
GRAD_BOUND = {
    "tiny": {"log1": 1e-5, "log0": 1e-5},        # measured 3.6e-6 / 3.6e-6  (|log-likelihood| <= 40)
    "cfg2": {"log1": 1.1e-3, "log0": 7.5e-4},    # measured 7.3e-4 / 5.0e-4  (<= 3911)
    "cfg3": {"log1": 7e-4, "log0": 7e-4},        # measured 4.7e-4 / 4.7e-4  (<= 3021)
    "cfg4": {"log1": 7.5e-4, "log0": 5e-5},      # measured 4.9e-4 / 2.5e-5  (<= 2861)
    "cfg5x4": {"log1": 1.5e-3, "log0": 1.5e-3},  # measured 9.7e-4 / 9.4e-4  (<= 7476)
}
VARIANTS = {"linear": {"OT_LATTICE": "linear"},
            "log1": {"OT_LATTICE": "log", "OT_FAST_MATH": "1"},
            "log0": {"OT_LATTICE": "log", "OT_FAST_MATH": "0"}}
RESULTS = []


def _batch(name):
    if name == "tiny":  # log-likelihoods of a few tens: float32 holds 1e-5 here
        w = synthetic.Workload("tiny", 6, (4, 9), (2, 4), 40, seed=77)
        n = w.n
    elif name == "cfg5x4":
        w, n = synthetic.CONFIGS["cfg5"], 4
    else:
        w = synthetic.CONFIGS[name]
        n = w.n
    T, U, tg = synthetic.make_lengths(w)
    T, U = T[:n].contiguous(), U[:n].contiguous()
    tg = tg[:n, :int(U.max())].contiguous()
    x = synthetic.make_utterance_logits(w, T, U, range(n), device="cpu")
    return w, x, tg, T, U


def _rel_to_one(a, b):
    return float(np.max(np.abs(a - b) / np.maximum(1.0, np.abs(b))))


@pytest.mark.parametrize("name", ["tiny", "cfg2", "cfg3", "cfg4", "cfg5x4"])
def test_cuda_path_against_the_reference_build(name, monkeypatch):
    if O.load_ref() is None:
        pytest.skip("oracle/_ref (the reference's own CPU build) is not present")
    w, x, tg, T, U = _batch(name)
    xn, tgn, Tn, Un = x.numpy(), tg.numpy(), T.numpy(), U.numpy()
    fl, mod = w.from_log_softmax, w.one_sym_per_frame
    band = O.band_mask(Tn, Un) if mod else np.ones(xn.shape[0], bool)

    # the reference's own build: scores + gradient, and its stages
    ref_scores, ref_grad = O.ref_loss(xn, tgn, Tn, Un, 0, fl, mod)
    st = O.ref_stages(xn, tgn, Tn, Un, 0, fl, mod)
    m = float(np.max(np.abs(ref_scores)))

    # the C port and the float64 restatement, for the table
    port = O.oracle_loss(xn, tgn, Tn, Un, 0, fl, mod)
    port_vs_ref = float(np.max(np.abs(port["grad"] - ref_grad)))
    del port
    x64 = xn.astype(np.float64)
    truth = O.oracle_loss(x64, tgn, Tn, Un, 0, fl, mod)
    del x64
    ref_vs_f64 = float(np.max(np.abs(ref_grad.astype(np.float64) - truth["grad"])))
    score_ref_vs_f64 = float(np.max(np.abs(ref_scores - truth["scores"]) / np.abs(truth["scores"])))
    truth_grad = truth["grad"]
    del truth

    dt, dT, dU = tg.to(DEV), T.to(DEV), U.to(DEV)
    row = {"config": name, "rows": int(xn.shape[0]), "V": int(xn.shape[1]), "max_abs_loglik": m,
           "port_vs_ref_grad": port_vs_ref, "ref_vs_f64_grad": ref_vs_f64,
           "ref_vs_f64_score_rel": score_ref_vs_f64}
    for variant, env in VARIANTS.items():
        monkeypatch.delenv("OT_FAST_MATH", raising=False)
        for k_, v_ in env.items():
            monkeypatch.setenv(k_, v_)
        dx = x.to(DEV)
        stg = ot.stage_outputs(dx, dt, dT, dU, 0, fl, mod)
        dx.requires_grad_(True)
        scores, grad = ot.compute_transducer_loss(dx, dt, dT, dU, 0, fl, mod)
        g = grad.detach().cpu().numpy()
        s = scores.cpu().numpy()
        e_score = float(np.max(np.abs(s - ref_scores) / np.abs(ref_scores)))
        e_alpha = _rel_to_one(stg["alpha"].cpu().numpy()[band], st["alpha"][band])
        e_beta = _rel_to_one(stg["beta"].cpu().numpy()[band], st["beta"][band])
        e_grad = float(np.max(np.abs(g - ref_grad)))
        e_truth = float(np.max(np.abs(g.astype(np.float64) - truth_grad)))
        row[variant] = {"score_rel": e_score, "alpha": e_alpha, "beta": e_beta,
                              "grad_vs_ref": e_grad, "grad_vs_f64": e_truth}
        del dx, stg, scores, grad, g
        torch.cuda.empty_cache()
    RESULTS.append(row)
    print("\nPARITY " + json.dumps(row))
    path = os.environ.get("OT_PARITY_REPORT")
    if path:
        with open(path, "w") as f:
            json.dump(RESULTS, f, indent=1)
    for variant in VARIANTS:
        r = row[variant]
        assert r["score_rel"] <= 1e-5, (name, variant, r)
        assert r["alpha"] <= 1e-5 and r["beta"] <= 1e-5, (name, variant, r)
        if name == "tiny":
            assert r["grad_vs_ref"] <= 1e-5, (name, variant, r)
        elif variant == "linear":
            # as far from the reference as the reference is from float64, and at most
            # half as far from float64 as the reference
            assert r["grad_vs_ref"] <= 1.25 * ref_vs_f64, (name, variant, r, ref_vs_f64)
            assert r["grad_vs_f64"] <= 0.5 * ref_vs_f64, (name, variant, r, ref_vs_f64)
        else:
            assert r["grad_vs_ref"] <= GRAD_BOUND[name][variant], (name, variant, r)
            # closer to the reference than the reference is to the float64 result
            assert r["grad_vs_ref"] <= ref_vs_f64, (name, variant, r, ref_vs_f64)
            # and no further from the float64 result than the reference itself (25 % slack)
            assert r["grad_vs_f64"] <= 1.25 * ref_vs_f64 + 1e-6, (name, variant, r, ref_vs_f64)
