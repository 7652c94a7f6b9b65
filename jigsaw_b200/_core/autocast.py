"""Autocast policy for hand-written autograd Functions.

``torch.autocast`` does not reach inside a custom ``autograd.Function``; layers apply
the policy themselves: matmul-like ops cast *down* to the autocast dtype, normalisation /
softmax / loss ops promote *up* to fp32.

Reference parity: jigsaw/_core/autocast.py:44-66, :83-107, :110-133.
"""

from __future__ import annotations

import torch


def _device_type(tensors: tuple[torch.Tensor | None, ...]) -> str | None:
    for t in tensors:
        if t is not None:
            return t.device.type
    return None


def autocast_dtype(device_type: str) -> torch.dtype | None:
    """Active autocast dtype for ``device_type`` or ``None`` when autocast is off."""
    if torch.is_autocast_enabled(device_type):
        return torch.get_autocast_dtype(device_type)
    return None


def cast_to_autocast_dtype(*tensors: torch.Tensor | None) -> tuple[torch.Tensor | None, ...]:
    """Cast to the active autocast dtype (identity when autocast is off; ``None`` kept)."""
    kind = _device_type(tensors)
    dt = autocast_dtype(kind) if kind is not None else None
    if dt is None:
        return tensors
    return tuple(None if t is None else t.to(dt) for t in tensors)


def promote_to_fp32_under_autocast(*tensors: torch.Tensor | None) -> tuple[torch.Tensor | None, ...]:
    """Promote half-precision tensors to fp32 while autocast is active (wider dtypes kept)."""
    kind = _device_type(tensors)
    if kind is None or autocast_dtype(kind) is None:
        return tensors
    return tuple(None if t is None else t.to(torch.promote_types(t.dtype, torch.float32)) for t in tensors)


def resolve_matmul_dtype(device: torch.device, *operands: torch.Tensor) -> torch.dtype:
    """Result dtype of a matmul: the autocast dtype if active, else the promoted operand dtype."""
    dt = autocast_dtype(device.type)
    if dt is not None:
        return dt
    out = operands[0].dtype
    for o in operands[1:]:
        out = torch.promote_types(out, o.dtype)
    return out
