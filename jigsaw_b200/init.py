"""Shard-aware parameter initialisation.

``torch.nn.init`` derives fan-in / fan-out from the tensor it fills.  A shard of a weight
would therefore be initialised with the wrong scale.  The four fan-based initialisers here
take the *global* (unsharded) shape, or the fans directly, so that a sharded layer draws
from the same distribution as the undivided torch layer.  Per-element initialisers are
re-exported unchanged.

Reference parity: jigsaw/init.py:15-40 (exports), :52-96 (fan resolution), :115-280.
"""

from __future__ import annotations

import math
from collections.abc import Sequence

import torch
from torch.nn.init import calculate_gain, constant_, normal_, ones_, trunc_normal_, uniform_, zeros_

__all__ = [
    "calculate_gain",
    "constant_",
    "kaiming_normal_",
    "kaiming_uniform_",
    "normal_",
    "ones_",
    "trunc_normal_",
    "uniform_",
    "xavier_normal_",
    "xavier_uniform_",
    "zeros_",
]


def _fans(
    tensor: torch.Tensor,
    global_shape: Sequence[int] | None,
    fan_in: int | None,
    fan_out: int | None,
) -> tuple[int, int]:
    """Fan-in / fan-out of the unsharded parameter (explicit fans win over ``global_shape``)."""
    shape = tuple(global_shape) if global_shape is not None else tuple(tensor.shape)
    if fan_in is None or fan_out is None:
        if len(shape) < 2:
            raise ValueError("Fan in and fan out can not be computed for tensor with fewer than 2 dimensions")
        receptive = math.prod(shape[2:]) if len(shape) > 2 else 1
        computed_in, computed_out = shape[1] * receptive, shape[0] * receptive
        fan_in = computed_in if fan_in is None else fan_in
        fan_out = computed_out if fan_out is None else fan_out
    return int(fan_in), int(fan_out)


def _pick(mode: str, fan_in: int, fan_out: int) -> int:
    mode = mode.lower()
    if mode not in ("fan_in", "fan_out"):
        raise ValueError(f"Mode {mode} not supported, please use one of fan_in, fan_out")
    return fan_in if mode == "fan_in" else fan_out


def kaiming_uniform_(
    tensor: torch.Tensor,
    a: float = 0,
    mode: str = "fan_in",
    nonlinearity: str = "leaky_relu",
    generator: torch.Generator | None = None,
    *,
    global_shape: Sequence[int] | None = None,
    fan_in: int | None = None,
    fan_out: int | None = None,
) -> torch.Tensor:
    """He-uniform fill with the fans of the unsharded parameter."""
    if 0 in tensor.shape:
        return tensor
    fi, fo = _fans(tensor, global_shape, fan_in, fan_out)
    std = calculate_gain(nonlinearity, a) / math.sqrt(_pick(mode, fi, fo))
    bound = math.sqrt(3.0) * std
    with torch.no_grad():
        return tensor.uniform_(-bound, bound, generator=generator)


def kaiming_normal_(
    tensor: torch.Tensor,
    a: float = 0,
    mode: str = "fan_in",
    nonlinearity: str = "leaky_relu",
    generator: torch.Generator | None = None,
    *,
    global_shape: Sequence[int] | None = None,
    fan_in: int | None = None,
    fan_out: int | None = None,
) -> torch.Tensor:
    """He-normal fill with the fans of the unsharded parameter."""
    if 0 in tensor.shape:
        return tensor
    fi, fo = _fans(tensor, global_shape, fan_in, fan_out)
    std = calculate_gain(nonlinearity, a) / math.sqrt(_pick(mode, fi, fo))
    with torch.no_grad():
        return tensor.normal_(0.0, std, generator=generator)


def xavier_uniform_(
    tensor: torch.Tensor,
    gain: float = 1.0,
    generator: torch.Generator | None = None,
    *,
    global_shape: Sequence[int] | None = None,
    fan_in: int | None = None,
    fan_out: int | None = None,
) -> torch.Tensor:
    """Glorot-uniform fill with the fans of the unsharded parameter."""
    fi, fo = _fans(tensor, global_shape, fan_in, fan_out)
    bound = math.sqrt(3.0) * gain * math.sqrt(2.0 / float(fi + fo))
    with torch.no_grad():
        return tensor.uniform_(-bound, bound, generator=generator)


def xavier_normal_(
    tensor: torch.Tensor,
    gain: float = 1.0,
    generator: torch.Generator | None = None,
    *,
    global_shape: Sequence[int] | None = None,
    fan_in: int | None = None,
    fan_out: int | None = None,
) -> torch.Tensor:
    """Glorot-normal fill with the fans of the unsharded parameter."""
    fi, fo = _fans(tensor, global_shape, fan_in, fan_out)
    std = gain * math.sqrt(2.0 / float(fi + fo))
    with torch.no_grad():
        return tensor.normal_(0.0, std, generator=generator)
