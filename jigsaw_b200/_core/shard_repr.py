"""``extra_repr`` helper: ``name=size`` for the process groups a layer is sharded over.

Reference parity: jigsaw/_core/shard_repr.py:15-41.
"""

from __future__ import annotations

from collections.abc import Sequence

import torch.distributed as dist


def _n(g: "dist.ProcessGroup | int | None") -> int:
    if isinstance(g, int):
        return g
    return 1 if g is None else g.size()


def shard_repr(**groups: "dist.ProcessGroup | Sequence[dist.ProcessGroup | None] | int | None") -> str:
    """E.g. ``shard_repr(spatial=(gh, gw), channel=gc)`` -> ``"spatial=(1, 2), channel=2"``."""
    out = []
    for name, g in groups.items():
        if isinstance(g, int):
            val: int | tuple[int, ...] = g
        elif g is None or isinstance(g, dist.ProcessGroup):
            val = _n(g)
        else:
            val = tuple(_n(x) for x in g)
        out.append(f"{name}={val}")
    return ", ".join(out)
