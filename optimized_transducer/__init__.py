"""``import optimized_transducer``: the reference's import name, served by the
sm_100a implementation in ``optimized_transducer_b200``.

The reference package exports ``transducer_loss`` and ``TransducerLoss`` and
carries ``__version__`` (optimized_transducer/python/optimized_transducer/
__init__.py:11 and setup.py:104-105 of the reference); so does this alias.  The
reference's check that the running PyTorch is the one it was built against
(``__init__.py:3-9``) has no counterpart: the C-ABI library does not link torch.
"""
from optimized_transducer_b200 import TransducerLoss, transducer_loss  # noqa: F401
from optimized_transducer_b200 import __version__  # noqa: F401

__all__ = ["TransducerLoss", "transducer_loss", "__version__"]
