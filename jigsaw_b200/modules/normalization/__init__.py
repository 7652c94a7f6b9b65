"""Normalisation layers whose statistics span a cut axis.

``DistributedLayerNorm`` normalises over a feature axis that is cut over the column group: each rank reduces
its slice to (count, mean, M2), the partial moments are merged over the group, and weight and bias are held as
slices.  ``DistributedGroupNorm`` cuts channels over a channel group (whole groups per rank, so no statistics
travel for that cut) and may also be cut in space, in which case the moments of a group are merged over the
spatial groups.  Both convert from and to their ``torch.nn`` counterparts and re-shard between meshes.

Reference parity: jigsaw/modules/normalization/__init__.py (two public names).
"""

from ..._core.public import set_module
from ._group_norm import DistributedGroupNorm
from ._layer_norm import DistributedLayerNorm

__all__ = ["DistributedGroupNorm", "DistributedLayerNorm"]

set_module(globals(), __all__)
