"""Permute with re-sharding."""

from ..._core.public import set_module
from ._permute import distributed_permute

__all__ = ["distributed_permute"]

set_module(globals(), __all__)
