"""Distributed loss functions and modules."""

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
