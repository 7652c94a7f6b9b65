"""``DistributedGroupNorm``: GroupNorm with channels (whole groups) over ``channel_group`` and
statistics reduced over the spatial groups the sample is tiled across.

Without a spatial split it calls ``F.group_norm`` directly.  Weight and bias hold the local
channel slice and are replicated over the spatial groups.

Reference parity: jigsaw/modules/normalization/_group_norm.py:27-392.
"""

from __future__ import annotations

from collections.abc import Sequence
from typing import Any

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ... import parallel
from ..._core.placement import gather_dim
from ..._core.shard_repr import shard_repr
from ._functional import distributed_group_norm


def _as_list(spatial_group: Any) -> list:
    if spatial_group is None:
        return []
    if isinstance(spatial_group, dist.ProcessGroup):
        return [spatial_group]
    return list(spatial_group)


class DistributedGroupNorm(torch.nn.Module):
    def __init__(
        self,
        num_groups: int,
        num_channels: int,
        device: torch.device | str,
        channel_group: dist.ProcessGroup | None = None,
        eps: float = 1e-5,
        affine: bool = True,
        bias: bool = True,
        dtype: torch.dtype | None = None,
        spatial_group: "dist.ProcessGroup | Sequence[dist.ProcessGroup | None] | None" = None,
    ) -> None:
        super().__init__()
        self.num_groups, self.num_channels = num_groups, num_channels
        self.device = torch.device(device)
        self.channel_group = channel_group
        self.spatial_groups = tuple(_as_list(spatial_group))
        self.eps, self.affine = eps, affine
        if num_channels % num_groups:
            raise ValueError("num_channels must be divisible by num_groups")
        self._resolve()
        if affine:
            self.weight = torch.nn.Parameter(torch.ones(self.local_channels, device=self.device, dtype=dtype))
            self.bias = torch.nn.Parameter(torch.zeros(self.local_channels, device=self.device, dtype=dtype)) if bias else None
        else:
            self.register_parameter("weight", None)
            self.register_parameter("bias", None)
        self._mark()

    def _resolve(self) -> None:
        G = 1 if self.channel_group is None else self.channel_group.size()
        if self.num_groups % G or self.num_channels % G:
            raise ValueError(
                f"num_groups={self.num_groups} and num_channels={self.num_channels} must be divisible by the "
                f"channel group size {G} so that no normalization group straddles two shards"
            )
        self.local_groups = self.num_groups // G
        self.local_channels = self.num_channels // G
        self._sync_groups = [g for g in self.spatial_groups if g is not None and g.size() > 1]

    def _mark(self) -> None:
        for p in self.parameters():
            if not parallel.replica_groups(p):
                parallel.mark_replicated(p, self._sync_groups)
        with torch.no_grad():
            for p in self.parameters():
                for g in reversed(self._sync_groups):
                    dist.broadcast(p.data, group_src=0, group=g)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        w, b = parallel.sync_grad(self.weight, self.bias)
        if x.is_cuda:
            from ...ops import norm_fused

            out = norm_fused.maybe_fused_group_norm(x, self.local_groups, w, b, list(self._sync_groups), self.eps)
            if out is not None:
                return out
        if not self._sync_groups:
            return F.group_norm(x, self.local_groups, w, b, self.eps)
        return distributed_group_norm(x, self.local_groups, w, b, self._sync_groups, self.eps)

    @classmethod
    def convert_to_jigsaw(
        cls, model: torch.nn.GroupNorm, process_mesh_dict: dict, device: torch.device | str, row_kw: str = "row",
        col_kw: str = "col", model_kw: str = "model", **kwargs: Any,
    ) -> "DistributedGroupNorm":
        layer = cls(
            model.num_groups, model.num_channels, device, process_mesh_dict[col_kw], eps=model.eps,
            affine=model.affine, bias=getattr(model, "bias", None) is not None,
            dtype=None if model.weight is None else model.weight.dtype,
            spatial_group=kwargs.get("spatial_group", process_mesh_dict[row_kw]),
        )
        layer._load_global(model.weight, model.bias)
        return layer

    def _load_global(self, weight: torch.Tensor | None, bias: torch.Tensor | None) -> None:
        r = 0 if self.channel_group is None else self.channel_group.rank()
        n = self.local_channels
        with torch.no_grad():
            if weight is not None and self.weight is not None:
                self.weight.data = weight.detach()[r * n : (r + 1) * n].clone().to(self.device)
            if bias is not None and self.bias is not None:
                self.bias.data = bias.detach()[r * n : (r + 1) * n].clone().to(self.device)

    def merge_weights(self, from_process_mesh: dict, row_kw: str = "row", col_kw: str = "col",
                      model_kw: str = "model") -> tuple[torch.Tensor | None, torch.Tensor | None]:
        """All-gather the slices over the channel group (``row_kw`` and ``model_kw`` are accepted for a uniform
        signature: the parameters are not cut over them)."""
        g = from_process_mesh[col_kw]
        with torch.no_grad():
            w = None if self.weight is None else gather_dim(self.weight.detach(), g, 0)
            b = None if self.bias is None else gather_dim(self.bias.detach(), g, 0)
        return w, b

    def convert_to_torch(self, process_mesh_dict: dict, row_kw: str = "row", col_kw: str = "col", model_kw: str = "model") -> torch.nn.GroupNorm:
        w, b = self.merge_weights(process_mesh_dict, col_kw=col_kw)
        layer = torch.nn.GroupNorm(self.num_groups, self.num_channels, eps=self.eps, affine=self.affine, device=self.device)
        if w is not None:
            layer.weight.data = w
        if b is not None:
            layer.bias.data = b
        elif self.affine:
            layer.bias.data.zero_()
        return layer

    def reshard_parameters(self, from_process_mesh: dict, to_process_mesh: dict, pm_row_key: str = "row",
                           pm_col_key: str = "col", pm_model_key: str = "model") -> None:
        w, b = self.merge_weights(from_process_mesh, col_kw=pm_col_key)
        self.channel_group = to_process_mesh[pm_col_key]
        self.spatial_groups = tuple(_as_list(to_process_mesh[pm_row_key]))
        self._resolve()
        if self.weight is not None:
            self.weight = torch.nn.Parameter(torch.empty(0, device=self.device, dtype=w.dtype))
        if self.bias is not None:
            self.bias = torch.nn.Parameter(torch.empty(0, device=self.device, dtype=b.dtype))
        self._load_global(w, b)
        self._mark()

    def shard_spec(self) -> dict:
        """Which dimension of which parameter is cut over which group (sharded checkpoints)."""
        cut = () if self.channel_group is None else ((0, self.channel_group),)
        return {"weight": cut, "bias": cut}

    @property
    def num_local_groups(self) -> int:
        """Normalisation groups held by this rank (the reference's name of ``local_groups``)."""
        return self.local_groups

    @property
    def num_local_channels(self) -> int:
        return self.local_channels

    def get_parameter_count(self) -> int:
        if not self.affine:
            return 0
        return self.num_channels * (2 if self.bias is not None else 1)

    def extra_repr(self) -> str:
        tiles = 1
        for g in self.spatial_groups:
            tiles *= 1 if g is None else g.size()
        return (f"{self.num_groups}, {self.num_channels}, eps={self.eps}, affine={self.affine}, bias={self.bias is not None}, "
                + shard_repr(spatial=tiles, channel=self.channel_group))
