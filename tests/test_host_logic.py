"""Host-side behaviour that needs no GPU: the metadata checks that mirror
ot::ComputeTransducerLoss (optimized_transducer/csrc/transducer-loss.cc:33-60),
the loud failure without a CUDA device, and the synthetic workloads."""
import pytest
import torch

import optimized_transducer_b200 as ot
from optimized_transducer_b200 import synthetic
from optimized_transducer_b200.transducer_loss import _validate


def _args(v=5):
    T = torch.tensor([2, 3], dtype=torch.int32)
    U = torch.tensor([1, 2], dtype=torch.int32)
    logits = torch.randn(int((T * (U + 1)).sum()), v)
    targets = torch.randint(1, v, (2, 2), dtype=torch.int32)
    return logits, targets, T, U


def test_public_surface_matches_the_reference():
    import inspect
    sig = inspect.signature(ot.transducer_loss)
    assert list(sig.parameters) == ["logits", "targets", "logit_lengths", "target_lengths",
                                    "blank", "from_log_softmax", "one_sym_per_frame", "reduction"]
    assert sig.parameters["one_sym_per_frame"].default is False
    assert sig.parameters["reduction"].default == "mean"
    m = ot.TransducerLoss(blank=0)  # the reference's module raises here
    assert m.reduction == "mean" and isinstance(ot.__version__, str)
    fsig = inspect.signature(ot.TransducerLoss.forward)
    assert list(fsig.parameters)[1:] == ["logits", "targets", "logit_lengths", "target_lengths",
                                         "from_log_softmax", "one_sym_per_frame"]


def test_no_cpu_fallback():
    logits, targets, T, U = _args()
    with pytest.raises(RuntimeError, match="CUDA devices only"):
        ot.transducer_loss(logits, targets, T, U, blank=0, from_log_softmax=False)


@pytest.mark.parametrize("mutate,match", [
    (lambda a: (a[0].to(torch.int32), a[1], a[2], a[3]), "scalar type Float"),
    (lambda a: (a[0], a[1].long(), a[2], a[3]), "targets to have scalar type Int"),
    (lambda a: (a[0], a[1], a[2].long(), a[3]), "logit_lengths to have scalar type Int"),
    (lambda a: (a[0].t().contiguous().t(), a[1], a[2], a[3]), "logits to be contiguous"),
    (lambda a: (a[0][0], a[1], a[2], a[3]), "logits to be 2-dimensional"),
    (lambda a: (a[0], a[1][0], a[2], a[3]), "targets to be 2-dimensional"),
    (lambda a: (a[0], a[1], a[2][:1], a[3]), "same size"),
])
def test_metadata_checks(mutate, match):
    with pytest.raises(RuntimeError, match=match):
        _validate(*mutate(_args()), 0)


def test_reduction_is_asserted_like_the_reference():
    logits, targets, T, U = _args()
    with pytest.raises(AssertionError):
        ot.transducer_loss(logits, targets, T, U, blank=0, from_log_softmax=False, reduction="none")


@pytest.mark.parametrize("name", sorted(synthetic.CONFIGS))
def test_synthetic_workloads_are_reproducible_and_in_range(name):
    w = synthetic.CONFIGS[name]
    T, U, tg = synthetic.make_lengths(w)
    T2, U2, tg2 = synthetic.make_lengths(w)
    assert torch.equal(T, T2) and torch.equal(U, U2) and torch.equal(tg, tg2)
    assert T.numel() == w.n and int(T.min()) >= w.t_range[0] and int(T.max()) <= w.t_range[1]
    assert int(U.max()) <= w.u_range[1] and tg.shape == (w.n, int(U.max()))
    assert int(tg.min()) >= 1 and int(tg.max()) < w.v
    if w.one_sym_per_frame:
        assert bool((U <= T - 1).all())


def test_synthetic_logits_shape():
    w = synthetic.CONFIGS["cfg1"]
    T, U, _ = synthetic.make_lengths(w)
    x = synthetic.make_logits(w, T, U)
    assert x.shape == (synthetic.num_rows(T, U), w.v) and x.dtype == torch.float32


def test_reference_import_names_are_served():
    """``optimized_transducer`` exports what the reference package exports
    (python/optimized_transducer/__init__.py:11 of the reference) and
    ``_optimized_transducer.compute_transducer_loss`` has the argument names of the
    reference's pybind function (python/csrc/optimized_transducer.cc:15-19)."""
    import inspect
    import _optimized_transducer
    import optimized_transducer
    assert optimized_transducer.transducer_loss is ot.transducer_loss
    assert optimized_transducer.TransducerLoss is ot.TransducerLoss
    assert isinstance(optimized_transducer.__version__, str)
    sig = inspect.signature(_optimized_transducer.compute_transducer_loss)
    assert list(sig.parameters) == ["logits", "targets", "logit_lengths", "target_lengths", "blank",
                                    "from_log_softmax", "one_sym_per_frame"]


def test_check_modes(monkeypatch):
    from optimized_transducer_b200 import _lib
    from optimized_transducer_b200.transducer_loss import _CHECK_FLAG, _check_mode
    for env, want in (("0", "off"), ("1", "deferred"), ("2", "strict")):
        monkeypatch.setenv("OT_CHECKS", env)
        assert _check_mode() == want
    monkeypatch.setenv("OT_CHECKS", "1")
    assert _check_mode("strict") == "strict"   # the default of the native-style entry points
    monkeypatch.delenv("OT_CHECKS")
    assert _check_mode() == "deferred"
    assert _CHECK_FLAG["deferred"] == _lib.REPORT_ERRORS and _CHECK_FLAG["strict"] == _lib.CHECK_INPUTS


def test_gradient_tile_of_the_logits_free_backward_has_16_byte_rows():
    """joiner_loss pads the bfloat16 gradient tile so that its rows are a multiple
    of 16 bytes (the library contractions that read it need that to stay on the
    tensor cores), to a multiple of 64 columns when that is nearly free."""
    from optimized_transducer_b200.transducer_loss import _padded_columns
    assert [_padded_columns(v) for v in (64, 500, 504, 5000, 20, 36, 1028)] == [64, 512, 504, 5000, 24, 40, 1032]
    for v in range(4, 7681, 4):
        vp = _padded_columns(v)
        assert v <= vp <= 7680 and vp % 8 == 0 and vp - v < 64
