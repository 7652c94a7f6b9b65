"""Distributed layers, losses, metrics and their configuration objects.

Reference parity: jigsaw/modules/__init__.py:61-112.
"""

from .._core.comm import CommOp
from .._core.public import set_module
from . import activation, attention, convolution, functional, linear, loss, metrics, normalization, permute, roll
from .activation import DistributedSoftmax
from .attention import Attention, DistributedAttention, RingAttentionConfig
from .convolution import (
    ConvNdConfig,
    ConvTransposeNdConfig,
    DistributedConv1d,
    DistributedConv2d,
    DistributedConv3d,
    DistributedConvTranspose1d,
    DistributedConvTranspose2d,
    DistributedConvTranspose3d,
)
from .linear import (
    DistributedLinear,
    DistributedMatMulXTW,
    DistributedMatMulXW,
    DistributedMatMulXWT,
    LinearConfig,
    MatMulXTW,
    MatMulXW,
    MatMulXWT,
)
from .loss import (
    DistributedBCELoss,
    DistributedBCEWithLogitsLoss,
    DistributedCrossEntropyLoss,
    DistributedL1Loss,
    DistributedMSELoss,
    DistributedNLLLoss,
    DistributedSmoothL1Loss,
)
from .metrics import DistributedSegmentationMetrics
from .normalization import DistributedGroupNorm, DistributedLayerNorm
from .roll import DistributedRoll, Roll, RollConfig

__all__ = [
    "Attention",
    "DistributedAttention",
    "DistributedConv1d",
    "DistributedConv2d",
    "DistributedConv3d",
    "DistributedConvTranspose1d",
    "DistributedConvTranspose2d",
    "DistributedConvTranspose3d",
    "DistributedGroupNorm",
    "DistributedLayerNorm",
    "DistributedLinear",
    "DistributedMatMulXTW",
    "DistributedMatMulXW",
    "DistributedMatMulXWT",
    "DistributedRoll",
    "DistributedSoftmax",
    "MatMulXTW",
    "MatMulXW",
    "MatMulXWT",
    "Roll",
    "DistributedBCELoss",
    "DistributedBCEWithLogitsLoss",
    "DistributedCrossEntropyLoss",
    "DistributedL1Loss",
    "DistributedMSELoss",
    "DistributedNLLLoss",
    "DistributedSmoothL1Loss",
    "DistributedSegmentationMetrics",
    "ConvNdConfig",
    "ConvTransposeNdConfig",
    "LinearConfig",
    "RingAttentionConfig",
    "RollConfig",
    "CommOp",
    "functional",
    "activation",
    "attention",
    "convolution",
    "linear",
    "loss",
    "metrics",
    "normalization",
    "permute",
    "roll",
]

set_module(globals(), [n for n in __all__ if n not in ("CommOp",)])
CommOp.__module__ = __name__
