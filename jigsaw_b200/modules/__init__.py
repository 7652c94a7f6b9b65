"""Distributed layers, losses, metrics and their configuration objects.

Each sub-package holds one family and documents it: ``linear`` (tensor-parallel linear layers and block
products), ``convolution`` (domain- and channel-parallel convolutions with halo exchange), ``attention`` (ring
and Ulysses sequence parallelism), ``normalization``, ``activation``, ``roll``, ``permute``, ``loss`` and
``metrics``; ``functional`` gathers the function forms.  The layer classes and configuration objects are also
importable from here, and ``CommOp`` names the transport of the neighbour exchanges that most of them accept as
``comm=``.  Every layer takes the process groups it is cut over as constructor arguments (for a spatial
axis, a loss, a metric, a norm's spatial cut, a softmax and the block products ``None`` means "not cut"), converts from and to its ``torch.nn`` counterpart, and can be moved between meshes with
``reshard_parameters``.

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

# everything imported above is public: the ten sub-packages, the layer and configuration classes, and CommOp
__all__ = sorted(name for name in dir() if not name.startswith("_") and name != "set_module")

set_module(globals(), [name for name in __all__ if name != "CommOp"])
CommOp.__module__ = __name__
