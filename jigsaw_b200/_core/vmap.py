"""Helpers for ``torch.vmap`` rules of custom autograd Functions (ensemble members as a leading axis).

Reference parity: jigsaw/_core/vmap.py:18-114.
"""

from __future__ import annotations

from typing import Any

import torch


def to_front(t: torch.Tensor | None, dim: int | None, batch_size: int) -> torch.Tensor | None:
    """Move the vmapped dimension to the front; unbatched tensors are expanded."""
    if t is None:
        return None
    if dim is None:
        return t.unsqueeze(0).expand(batch_size, *t.shape)
    return t.movedim(dim, 0)


def batch_size_of(info: Any) -> int:
    return int(info.batch_size)


def ensure_not_nested(info: Any) -> None:
    """Only one level of vmap is supported by the distributed rules."""
    if getattr(info, "randomness", None) == "different":
        return
    level = getattr(torch._C._functorch, "maybe_current_level", lambda: None)()
    if level is not None and level > 1:
        raise NotImplementedError("nested torch.vmap over distributed layers is not supported")
