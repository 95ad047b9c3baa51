"""B200-native (sm_100a) transducer loss, a drop-in for the loss path of
csukuangfj/optimized_transducer:

    import optimized_transducer_b200 as optimized_transducer
    loss = optimized_transducer.transducer_loss(logits, targets, logit_lengths,
                                                target_lengths, blank=0,
                                                from_log_softmax=False)
"""
from .transducer_loss import (PerUtteranceLossFunction, TransducerLoss,  # noqa: F401
                              TransducerLossFunction, check_inputs, compute_transducer_loss,
                              joiner_loss, joiner_scores, stage_outputs, transducer_loss,
                              transducer_loss_and_grad, transducer_loss_per_utterance)

from .packing import pack_joiner_input, pack_padded, rnnt_loss, unpack_to_padded  # noqa: F401,E402

__version__ = "0.1.0"
__all__ = ["transducer_loss", "TransducerLoss", "TransducerLossFunction",
           "compute_transducer_loss", "stage_outputs", "transducer_loss_per_utterance",
           "transducer_loss_and_grad",
           "PerUtteranceLossFunction", "check_inputs", "joiner_scores", "joiner_loss", "pack_joiner_input", "pack_padded",
           "unpack_to_padded", "rnnt_loss", "__version__"]
