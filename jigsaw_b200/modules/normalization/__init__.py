"""Normalisation layers over sharded dimensions."""

from ..._core.public import set_module
from ._group_norm import DistributedGroupNorm
from ._layer_norm import DistributedLayerNorm

__all__ = ["DistributedGroupNorm", "DistributedLayerNorm"]

set_module(globals(), __all__)
