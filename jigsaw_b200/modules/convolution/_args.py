"""Constructor-argument normalisation shared by the convolution layers.

Reference parity: jigsaw/modules/convolution/_common/arg_norm.py:8-78,
jigsaw/modules/convolution/_common/channel_comm.py:62-115 (group / channel validation).
"""

from __future__ import annotations

from collections.abc import Sequence

import torch
import torch.distributed as dist

from ..._core.comm import CommOp, resolve_comm_op


def ntuple(x: int | Sequence[int], n: int) -> tuple[int, ...]:
    """An int or 1-tuple is broadcast to ``n`` axes; an ``n``-tuple is kept; else ``ValueError``."""
    if isinstance(x, int):
        return (x,) * n
    x = tuple(x)
    if len(x) == 1:
        return (x[0],) * n
    if len(x) != n:
        raise ValueError(f"expected an int or a tuple of 1 or {n} entries (one per spatial axis); got {x!r}.")
    return x


def resolve_padding(
    padding: int | str | Sequence[int], kernel: tuple[int, ...], stride: tuple[int, ...], dilation: tuple[int, ...]
) -> str | tuple[int, ...]:
    """Integers per axis; ``"same"`` is kept as a string only when an axis pads asymmetrically."""
    n = len(kernel)
    if not isinstance(padding, str):
        return ntuple(padding, n)
    if padding == "valid":
        return (0,) * n
    if padding != "same":
        raise ValueError(f"Invalid padding string {padding!r}, should be one of ('valid', 'same')")
    if any(s != 1 for s in stride):
        raise ValueError("padding='same' is not supported for strided convolutions")
    total = [d * (k - 1) for k, d in zip(kernel, dilation)]
    if any(t % 2 for t in total):
        return "same"
    return tuple(t // 2 for t in total)


def spatial_groups_tuple(
    spatial_group: "dist.ProcessGroup | Sequence[dist.ProcessGroup | None] | None", n: int
) -> tuple[dist.ProcessGroup | None, ...]:
    """One entry per spatial axis; a single group splits the LAST axis only."""
    if spatial_group is None:
        return (None,) * n
    if isinstance(spatial_group, dist.ProcessGroup):
        return (None,) * (n - 1) + (spatial_group,)
    groups = tuple(spatial_group)
    if len(groups) != n:
        raise ValueError(
            f"spatial_group as a sequence must have {n} entries (one per spatial axis, innermost last); "
            f"got {len(groups)}."
        )
    return groups


def resolve_conv_groups(groups: int, cin: int, cout: int, G: int) -> tuple[bool, int]:
    """Validate ``groups`` against the channel counts and the channel group size ``G``.

    Returns ``(channel_local, groups_local)``: when ``groups`` is a multiple of ``G`` every
    rank owns whole convolution groups and needs no channel communication.
    """
    if groups < 1:
        raise ValueError(f"groups must be >= 1, got {groups}")
    if cin % groups or cout % groups:
        raise ValueError(f"in_channels ({cin}) and out_channels ({cout}) must both be divisible by groups ({groups})")
    if cin % G or cout % G:
        raise ValueError(
            f"in_channels ({cin}) and out_channels ({cout}) must both be divisible by the channel group size ({G})"
        )
    if groups != 1 and groups % G != 0:
        raise NotImplementedError(
            "Distributed grouped convolution needs groups == 1 or groups to be a multiple of the "
            f"channel-parallel group size ({G}); got groups={groups}."
        )
    local = groups % G == 0
    return local, (groups // G if local else 1)


CHANNEL_COMMS = ("all_gather", *[m.value for m in CommOp])


def resolve_channel_comm(channel_comm: CommOp | str, device: torch.device | str) -> str:
    """``"all_gather"`` or a resolved :class:`CommOp` value (ring of partial convolutions)."""
    if channel_comm == "all_gather":
        return "all_gather"
    if str(channel_comm).lower() not in {m.value for m in CommOp}:
        raise ValueError(f"channel_comm must be 'auto' or one of {list(CHANNEL_COMMS)}, got {channel_comm!r}")
    return resolve_comm_op(channel_comm, torch.device(device)).value


def layer_key(channel_group: dist.ProcessGroup, bias: object, kernel: Sequence[int], stride: Sequence[int], groups: int) -> dict:
    """Properties a conv config depends on; a config built for other values is rejected."""
    return {
        "n_spatial": len(kernel),
        "bias": bias is not None,
        "kernel_size == stride": tuple(kernel) == tuple(stride),
        "groups": groups,
        "channel group size": channel_group.size(),
    }
