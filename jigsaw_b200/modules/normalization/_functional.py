"""LayerNorm / GroupNorm math over sharded dimensions.

LayerNorm: the normalised (last) dimension is split over ``col_group``; each row's mean and
centred second moment need a sum over the group.  GroupNorm: whole channel groups live on
one channel rank, but the spatial extent of a sample is tiled over the spatial groups, so
per-(sample, group) count/sum and centred sum of squares are summed over those.  Both are
written with differentiable all-reduces (sum forward, sum backward) so the distributed
backward (two more small reductions) is derived by autograd.  fp32 under autocast.

On CUDA the LayerNorm forward/backward take the fused kernels of ``jigsaw_b200.ops``
(local statistics, peer exchange and normalisation in one launch) when available.

Reference parity: jigsaw/modules/normalization/_functional.py:13-177 (LayerNorm), :187-308
(no-affine), :317-468 (GroupNorm).
"""

from __future__ import annotations

from collections.abc import Sequence

import torch
import torch.distributed as dist

from ..._core.autocast import promote_to_fp32_under_autocast
from ..._core.collectives import all_reduce_sum


def distributed_layer_norm(
    x: torch.Tensor,
    weight: torch.Tensor | None,
    bias: torch.Tensor | None,
    col_group: dist.ProcessGroup | None,
    eps: float,
) -> torch.Tensor:
    """Normalise the last dimension of ``x`` (split over ``col_group``) and apply the local
    shard of the affine parameters."""
    x, weight, bias = promote_to_fp32_under_autocast(x, weight, bias)
    parts = 1 if col_group is None else col_group.size()
    c_global = x.shape[-1] * parts
    mean = all_reduce_sum(x.sum(dim=-1, keepdim=True), col_group) / c_global
    centred = x - mean
    var = all_reduce_sum((centred * centred).sum(dim=-1, keepdim=True), col_group) / c_global
    y = centred * torch.rsqrt(var + eps)
    if weight is not None:
        y = y * weight
    if bias is not None:
        y = y + bias
    return y


def distributed_group_norm(
    x: torch.Tensor,
    num_groups_local: int,
    weight: torch.Tensor | None,
    bias: torch.Tensor | None,
    spatial_groups: Sequence[dist.ProcessGroup],
    eps: float,
) -> torch.Tensor:
    """GroupNorm of ``x`` ``(N, C_local, *spatial_local)`` with statistics reduced over the
    spatial groups.  ``num_groups_local`` normalisation groups live on this channel rank."""
    x, weight, bias = promote_to_fp32_under_autocast(x, weight, bias)
    n, c = x.shape[0], x.shape[1]
    xg = x.reshape(n, num_groups_local, -1)
    world = 1
    for g in spatial_groups:
        world *= g.size()
    count = xg.shape[-1] * world
    mean = all_reduce_sum(xg.sum(dim=-1, keepdim=True), spatial_groups) / count
    centred = xg - mean
    var = all_reduce_sum((centred * centred).sum(dim=-1, keepdim=True), spatial_groups) / count
    y = (centred * torch.rsqrt(var + eps)).reshape(x.shape)
    shape = (1, c) + (1,) * (x.dim() - 2)
    if weight is not None:
        y = y * weight.view(shape)
    if bias is not None:
        y = y + bias.view(shape)
    return y
