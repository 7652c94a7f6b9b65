"""Building blocks shared by the model families: replicated plain layers and the
column-parallel variants of linear / layer norm for tiled (domain-parallel) token maps.

A *tile context* describes how a feature map is laid out: its spatial axes are cut over the
``spatial`` groups (weights are replicated over those, gradients summed), its channel axis
over ``col`` (weights are split over that one).

Reference parity: the ``replicate`` helper of examples/swin.py:71-82 (broadcast from rank 0,
``mark_replicated`` over the tile groups, gradients summed through ``synced_parameters``).
"""

from __future__ import annotations

from collections.abc import Sequence
from dataclasses import dataclass

import torch
import torch.distributed as dist
from torch import nn

from .. import parallel
from ..modules import DistributedLayerNorm, DistributedLinear


@dataclass
class TileContext:
    spatial: tuple[dist.ProcessGroup | None, ...]
    col: dist.ProcessGroup | None
    device: torch.device
    dtype: torch.dtype = torch.float32

    @property
    def live_spatial(self) -> list[dist.ProcessGroup]:
        return [g for g in self.spatial if g is not None and g.size() > 1]

    @property
    def col_size(self) -> int:
        return 1 if self.col is None else self.col.size()

    @property
    def col_rank(self) -> int:
        return 0 if self.col is None else self.col.rank()


def mark_all(module: nn.Module, groups: Sequence[dist.ProcessGroup]) -> nn.Module:
    """Mark every parameter of ``module`` replicated over ``groups`` (in addition to marks it
    already has) and make the replicas equal."""
    groups = [g for g in groups if g is not None and g.size() > 1]
    if groups:
        for p in module.parameters():
            parallel.mark_replicated(p, groups, extend=True)
        parallel.broadcast_replicas(module)
    return module



class ReplicatedLinear(nn.Linear):
    """``nn.Linear`` replicated over the tile groups (same parameter names as the sharded layer,
    so checkpoints do not depend on the mesh)."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        w, b = parallel.sync_grad(self.weight, self.bias)
        if x.is_cuda:
            from ..ops import linear_fused

            out = linear_fused.maybe_fused_linear(x, w, b)      # tcgen05 GEMM under bf16 autocast
            if out is not None:
                return out
        return torch.nn.functional.linear(x, w, b)


class ReplicatedLayerNorm(nn.LayerNorm):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        w, b = parallel.sync_grad(self.weight, self.bias)
        if x.is_cuda and len(self.normalized_shape) == 1:
            from ..ops import norm_fused

            out = norm_fused.maybe_fused_layer_norm(x, w, b, None, self.eps)
            if out is not None:
                return out
        return torch.nn.functional.layer_norm(x, self.normalized_shape, w, b, self.eps)


def tile_linear(ctx: TileContext, in_dim: int, out_dim: int, bias: bool = True) -> nn.Module:
    """Linear layer on the last axis of a tiled map: plain + replicated when channels are whole,
    column-parallel (input and output features over ``col``) otherwise."""
    if ctx.col_size == 1:
        return mark_all(ReplicatedLinear(in_dim, out_dim, bias=bias, device=ctx.device, dtype=ctx.dtype), ctx.live_spatial)
    live = ctx.live_spatial
    # the layer marks over one group itself (a size-1 axis when no spatial axis is split) ...
    row = live[0] if live else next(g for g in ctx.spatial if g is not None)
    layer = DistributedLinear(in_dim, out_dim, ctx.device, ctx.col, row, ctx.col, bias=bias, dtype=ctx.dtype)
    if not live:
        return layer
    return mark_all(layer, live)                 # ... the remaining tile groups are added here


def tile_layer_norm(ctx: TileContext, dim: int) -> nn.Module:
    if ctx.col_size == 1:
        return mark_all(ReplicatedLayerNorm(dim, device=ctx.device, dtype=ctx.dtype), ctx.live_spatial)
    live = ctx.live_spatial
    layer = DistributedLayerNorm(dim, None, ctx.device, live[0] if live else None, ctx.col, dtype=ctx.dtype)
    return mark_all(layer, live)
