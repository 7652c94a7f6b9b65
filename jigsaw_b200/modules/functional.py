"""Functional forms of the distributed operations, gathered in one namespace in the manner of
``torch.nn.functional``.

==================================================  ==============================================================
``distributed_argmax``                              global index of the maximum along a cut axis
``distributed_log_softmax``                         log-softmax along a cut axis
``distributed_cross_entropy``                       cross entropy, class axis and / or space cut
``distributed_nll_loss``                            negative log-likelihood on log-probabilities
``distributed_binary_cross_entropy``                BCE on probabilities
``distributed_binary_cross_entropy_with_logits``    BCE on logits, with ``pos_weight``
``distributed_l1_loss`` / ``distributed_mse_loss``  mean or summed absolute / squared error over all tiles
``distributed_smooth_l1_loss``                      Huber-type loss with ``beta``
``redundant_all_reduce``                            sum of a value held identically by several ranks
``distributed_confusion_matrix``                    class-by-class counts over all tiles
``confusion_to_metrics``                            accuracy, IoU, Dice, precision, recall from the counts
``distributed_permute``                             ``permute`` that also moves the cut from one axis to another
==================================================  ==============================================================

Reference parity: jigsaw/modules/functional.py:19-37.
"""

from .activation import distributed_argmax, distributed_log_softmax
from .loss import (
    distributed_binary_cross_entropy,
    distributed_binary_cross_entropy_with_logits,
    distributed_cross_entropy,
    distributed_l1_loss,
    distributed_mse_loss,
    distributed_nll_loss,
    distributed_smooth_l1_loss,
    redundant_all_reduce,
)
from .metrics import confusion_to_metrics, distributed_confusion_matrix
from .permute import distributed_permute

__all__ = [
    "confusion_to_metrics",
    "distributed_argmax",
    "distributed_binary_cross_entropy",
    "distributed_binary_cross_entropy_with_logits",
    "distributed_confusion_matrix",
    "distributed_cross_entropy",
    "distributed_l1_loss",
    "distributed_log_softmax",
    "distributed_mse_loss",
    "distributed_nll_loss",
    "distributed_permute",
    "distributed_smooth_l1_loss",
    "redundant_all_reduce",
]
