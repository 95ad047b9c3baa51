"""``import _optimized_transducer``: the name of the reference's native module
(``PYBIND11_MODULE(_optimized_transducer, m)``,
optimized_transducer/python/csrc/optimized_transducer.cc:12-19 of the reference),
for callers of that private module.  Its one function

    compute_transducer_loss(logits, targets, logit_lengths, target_lengths,
                            blank, from_log_softmax, one_sym_per_frame)
        -> (scores, grad or None)

has the reference's argument names and return convention: ``scores[b]`` is
``log P(y_b | x_b)``; the gradient of ``-scores.sum()`` is returned only if
``logits.requires_grad``, and with ``from_log_softmax=False`` it is written over
``logits`` (the returned tensor shares its memory).  CUDA tensors only.
"""
from optimized_transducer_b200.transducer_loss import compute_transducer_loss  # noqa: F401

__all__ = ["compute_transducer_loss"]
