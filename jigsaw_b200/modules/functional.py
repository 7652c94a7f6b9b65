"""Functional forms of the distributed operations.

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
