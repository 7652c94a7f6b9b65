"""Roll of tiled tensors."""

from ..._core.public import set_module
from ._roll import DistributedRoll, Roll, RollConfig

__all__ = ["DistributedRoll", "Roll", "RollConfig"]

set_module(globals(), __all__)
