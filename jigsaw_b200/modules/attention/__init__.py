"""Attention layers and their sequence-parallel policies."""

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
