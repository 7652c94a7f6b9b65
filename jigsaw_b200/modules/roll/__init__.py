"""``torch.roll`` for tensors that are cut into tiles over process groups.

A shift moves whole tiles between ranks plus a remainder inside the tile, so a rank receives pieces from at most
two neighbours per rolled axis.  ``Roll`` is ``torch.roll`` as a module, which the converter replaces
by ``DistributedRoll``, the module over several cut axes (the shifted windows of Swin use it); ``RollConfig``
holds its transport option.  Shifts larger than a tile, negative shifts, gradients and ``vmap`` are supported.

Reference parity: jigsaw/modules/roll/__init__.py (three public names).
"""

from ..._core.public import set_module
from ._roll import DistributedRoll, Roll, RollConfig

__all__ = ["DistributedRoll", "Roll", "RollConfig"]

set_module(globals(), __all__)
