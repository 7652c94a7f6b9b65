"""``extra_repr`` helper: ``name=size`` for the process groups a layer is sharded over.

A layer's ``repr`` should say how it is cut without a reader having to look the groups up: ``spatial=(1, 2),
channel=2`` reads "not cut along the first spatial axis, two tiles along the second, channels over two ranks".

Reference parity: jigsaw/_core/shard_repr.py:15-41.
"""

from __future__ import annotations

from collections.abc import Sequence

import torch.distributed as dist


def _parts(entry: object) -> "int | tuple":
    """Ranks that ``entry`` cuts over: a group's size, 1 for ``None`` (not cut), a number as it is, and a tuple
    of those for a sequence (one entry per axis)."""
    if entry is None:
        return 1
    if isinstance(entry, int):
        return entry
    if isinstance(entry, dist.ProcessGroup) or callable(getattr(entry, "size", None)):      # a group, or a stand-in for one
        return entry.size()
    return tuple(_parts(e) for e in entry)


def shard_repr(**groups: "dist.ProcessGroup | Sequence[dist.ProcessGroup | None] | int | None") -> str:
    """E.g. ``shard_repr(spatial=(gh, gw), channel=gc)`` -> ``"spatial=(1, 2), channel=2"``."""
    return ", ".join(f"{name}={_parts(entry)}" for name, entry in groups.items())
