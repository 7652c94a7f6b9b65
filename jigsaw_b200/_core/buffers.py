"""Grow-only cache of communication buffers keyed by call site.

A buffer is identified by (file, line) of the caller plus device, dtype and a
caller-chosen index; it only ever grows and is handed out as a view of the requested
shape.  Contract: consume a buffer before the same call site asks for it again.

Reference parity: jigsaw/_core/buffers.py:17-73.
"""

from __future__ import annotations

import math
import sys
from collections.abc import Sequence

import torch

_cache: dict[tuple, torch.Tensor] = {}


def preallocated_buffer(
    shape: Sequence[int], dtype: torch.dtype, device: torch.device | str, index: int = 0, *, zero: bool = False, depth: int = 1
) -> torch.Tensor:
    """Return a cached buffer of ``shape`` for the calling line (``depth`` frames up)."""
    frame = sys._getframe(depth)
    device = torch.device(device)
    key = (frame.f_code.co_filename, frame.f_lineno, str(device), dtype, index)
    n = math.prod(shape)
    buf = _cache.get(key)
    if buf is None or buf.numel() < n:
        buf = torch.zeros(n, dtype=dtype, device=device)
        _cache[key] = buf
    elif zero:
        buf[:n].zero_()
    return buf[:n].view(*shape)


def clear_preallocated_buffers() -> None:
    """Drop every cached buffer (e.g. between phases with very different shapes)."""
    _cache.clear()
