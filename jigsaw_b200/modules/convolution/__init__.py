"""Distributed convolutions (see :mod:`._conv`).

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
