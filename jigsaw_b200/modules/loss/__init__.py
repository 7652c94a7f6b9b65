"""Losses for predictions and targets that are cut over ranks.

Each loss reduces its local tile and then sums numerator and denominator over the groups that hold the other
tiles, so ``reduction="mean"`` is the mean over the whole tensor and not the mean of per-rank means.  The
classification losses also accept a class axis cut over a channel group: the log-sum-exp is merged over that
group and the picked logit comes from the rank that owns the target class.  ``weight``, ``ignore_index`` and
``label_smoothing`` follow ``torch.nn.functional``.  ``redundant_all_reduce`` sums a value that several ranks
hold identically and gives each of them the gradient of the one copy.

Reference parity: jigsaw/modules/loss/__init__.py (seven modules, eight functions).
"""

from ..._core.public import set_module
from ._functional import (
    distributed_binary_cross_entropy,
    distributed_binary_cross_entropy_with_logits,
    distributed_cross_entropy,
    distributed_l1_loss,
    distributed_mse_loss,
    distributed_nll_loss,
    distributed_smooth_l1_loss,
    redundant_all_reduce,
)
from ._modules import (
    DistributedBCELoss,
    DistributedBCEWithLogitsLoss,
    DistributedCrossEntropyLoss,
    DistributedL1Loss,
    DistributedMSELoss,
    DistributedNLLLoss,
    DistributedSmoothL1Loss,
)

__all__ = [
    "DistributedBCELoss",
    "DistributedBCEWithLogitsLoss",
    "DistributedCrossEntropyLoss",
    "DistributedL1Loss",
    "DistributedMSELoss",
    "DistributedNLLLoss",
    "DistributedSmoothL1Loss",
    "distributed_binary_cross_entropy",
    "distributed_binary_cross_entropy_with_logits",
    "distributed_cross_entropy",
    "distributed_l1_loss",
    "distributed_mse_loss",
    "distributed_nll_loss",
    "distributed_smooth_l1_loss",
    "redundant_all_reduce",
]

set_module(globals(), __all__)
