"""Domain- and channel-parallel convolutions in one, two and three dimensions.

The spatial axes of the activation are cut over up to three process groups and the channels over a fourth; a
layer exchanges just the halo its kernel, stride, dilation and padding need, runs the local convolution and sums
partial results over the channel group.  The transposed layers scatter their overhang back to the neighbours
instead.  ``ConvNdConfig`` / ``ConvTransposeNdConfig`` record the layer's geometry, how the channel sum travels
(``channel_comm``) and whether grouped channels stay on one rank.  On CUDA the 3x3
64-channel bf16 case runs on tcgen05 kernels that read the halo from the neighbours' memory.

Reference parity: jigsaw/modules/convolution/__init__.py (eight public names).
"""

from ..._core.public import set_module
from ._config import ConvNdConfig, ConvTransposeNdConfig
from ._conv import (
    DistributedConv1d,
    DistributedConv2d,
    DistributedConv3d,
    DistributedConvTranspose1d,
    DistributedConvTranspose2d,
    DistributedConvTranspose3d,
)

__all__ = [
    "ConvNdConfig",
    "ConvTransposeNdConfig",
    "DistributedConv1d",
    "DistributedConv2d",
    "DistributedConv3d",
    "DistributedConvTranspose1d",
    "DistributedConvTranspose2d",
    "DistributedConvTranspose3d",
]

set_module(globals(), __all__)
