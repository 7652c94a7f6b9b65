"""Ulysses sequence parallelism: one all-to-all turns the sequence shard into a head shard,
dense attention runs on the full sequence, the inverse all-to-all restores the layout.

Tensors are ``bshd``.  The all-to-all is the differentiable ``all_to_all_dims`` (its backward
is the inverse exchange), so no hand-written backward is needed.  The hierarchical variant
runs Ulysses inside intra groups and a K/V ring across them.

On CUDA each exchange is one peer-memory all-to-all kernel (``jigsaw_b200.ops.exchange_fused``);
``jigsaw_b200.ops.ulysses_fused`` holds opt-in forms that fuse the exchanges into the projections
next to them.

Reference parity: jigsaw/modules/attention/_functional/ulysses.py:19-63 (all-to-alls),
:66-144 (ulysses_attention), :147-180 (hierarchical).
"""

from __future__ import annotations

from collections.abc import Callable

import torch
import torch.distributed as dist

from ..._core.collectives import all_to_all_dims
from ._config import RingAttentionConfig
from ._ring import ring_attention


def seq_to_heads(t: torch.Tensor, group: dist.ProcessGroup) -> torch.Tensor:
    """``(..., s/P, h, d)`` -> ``(..., s, h/P, d)``."""
    return all_to_all_dims(t, group, split_dim=-2, cat_dim=-3)


def heads_to_seq(t: torch.Tensor, group: dist.ProcessGroup) -> torch.Tensor:
    """``(..., s, h/P, d)`` -> ``(..., s/P, h, d)``."""
    return all_to_all_dims(t, group, split_dim=-3, cat_dim=-2)


def ulysses_attention(
    qkv: torch.Tensor, group: dist.ProcessGroup, dense: Callable[[torch.Tensor, torch.Tensor, torch.Tensor], torch.Tensor]
) -> torch.Tensor:
    """``qkv``: stacked ``(3, ..., s/P, h, d)``; ``dense(q, k, v)`` works in ``(..., h, s, d)``.
    Returns ``(..., s/P, h, d)``."""
    full = seq_to_heads(qkv, group)                       # one exchange for q, k and v together
    q, k, v = (t.transpose(-3, -2) for t in full.unbind(0))
    out = dense(q, k, v).transpose(-3, -2)                # (..., s, h/P, d)
    return heads_to_seq(out.contiguous(), group)


def hierarchical_ulysses_attention(
    qkv: torch.Tensor, intra: dist.ProcessGroup, inter: dist.ProcessGroup, scale: float, cfg: RingAttentionConfig,
    dropout_p: float = 0.0,
) -> torch.Tensor:
    """Ulysses inside ``intra``; the resulting (intra-complete) sequences attend across
    ``inter`` with a K/V ring."""
    full = seq_to_heads(qkv, intra)
    q, k, v = (t.transpose(-3, -2).contiguous() for t in full.unbind(0))
    out = ring_attention(q, k, v, scale, inter, cfg, dropout_p).transpose(-3, -2)
    return heads_to_seq(out.contiguous(), intra)
