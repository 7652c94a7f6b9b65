"""Multi-head attention with sequence parallelism.

``Attention`` is the single-device layer, ``DistributedAttention`` cuts the sequence over the row group and the
heads over the column group.  K/V chunks travel around the row group by the schedule ``SendOp`` names (ring,
owner broadcast, two-level hybrids); ``SendForward`` / ``SaveBackward`` / ``SaveScope`` / ``Offload`` /
``SendBackward`` choose what travels, what is kept for the backward pass and where, and how dK/dV return.
``ulysses=True`` re-shards from sequence to heads with two all-to-alls instead.  ``AttnBackend`` picks the
attention core; ``JIGSAW_TE_AVAILABLE`` tells whether TransformerEngine was found.

Reference parity: jigsaw/modules/attention/__init__.py.
"""

from ..._core.public import set_module
from ._attention import Attention, DistributedAttention
from ._config import (
    JIGSAW_TE_AVAILABLE,
    AttnBackend,
    Offload,
    RingAttentionConfig,
    SaveBackward,
    SaveScope,
    SendBackward,
    SendForward,
    SendOp,
)

__all__ = [
    "Attention",
    "AttnBackend",
    "DistributedAttention",
    "JIGSAW_TE_AVAILABLE",
    "Offload",
    "RingAttentionConfig",
    "SaveBackward",
    "SaveScope",
    "SendBackward",
    "SendForward",
    "SendOp",
]

set_module(globals(), __all__)
