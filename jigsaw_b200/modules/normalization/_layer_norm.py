"""``DistributedLayerNorm``: LayerNorm over a feature dimension split across ``col_group``.

Weight and bias hold the local ``C / col`` slice, are replicated (marked, broadcast) over
``row_group`` and get their gradients summed over it by ``sync_grad``.  Only a single
trailing normalised dimension is supported.

Reference parity: jigsaw/modules/normalization/_layer_norm.py:15-368.
"""

from __future__ import annotations

from typing import Any

import torch
import torch.distributed as dist

from ... import parallel
from ..._core.placement import check_divisible, gather_dim
from ..._core.shard_repr import shard_repr
from ._functional import distributed_layer_norm


class DistributedLayerNorm(torch.nn.Module):
    def __init__(
        self,
        normalized_dim: int,
        local_rank: int | None,
        device: torch.device | str,
        row_group: dist.ProcessGroup | None,
        col_group: dist.ProcessGroup | None,
        eps: float = 1e-5,
        elementwise_affine: bool = True,
        bias: bool = True,
        dtype: torch.dtype | None = None,
    ) -> None:
        super().__init__()
        if not isinstance(normalized_dim, int):
            if len(tuple(normalized_dim)) != 1:
                raise NotImplementedError("DistributedLayerNorm normalizes a single trailing dimension only")
            normalized_dim = int(tuple(normalized_dim)[0])
        self.normalized_dim = normalized_dim
        self.local_rank = local_rank                      # kept as given; the layer takes its place from the groups
        self.device = torch.device(device)
        self.row_group, self.col_group = row_group, col_group
        self.eps = eps
        self.elementwise_affine = elementwise_affine
        parts = 1 if col_group is None else col_group.size()
        local = check_divisible(normalized_dim, parts, "normalized_dim")
        if elementwise_affine:
            self.weight = torch.nn.Parameter(torch.ones(local, device=self.device, dtype=dtype))
            self.bias = torch.nn.Parameter(torch.zeros(local, device=self.device, dtype=dtype)) if bias else None
        else:
            self.register_parameter("weight", None)
            self.register_parameter("bias", None)
        self._mark()

    # the reference names the same things after what the groups cut (tokens, channels)
    @property
    def spatial_group(self) -> dist.ProcessGroup | None:
        return self.row_group

    @property
    def channel_group(self) -> dist.ProcessGroup | None:
        return self.col_group

    @property
    def local_dim(self) -> int:
        """Features of the normalised axis held by this rank."""
        return self.normalized_dim // (1 if self.col_group is None else self.col_group.size())

    def _mark(self) -> None:
        for p in self.parameters():
            if not parallel.replica_groups(p):
                parallel.mark_replicated(p, [self.row_group])
        with torch.no_grad():
            if self.row_group is not None and self.row_group.size() > 1:
                for p in self.parameters():
                    dist.broadcast(p.data, group_src=0, group=self.row_group)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        w, b = parallel.sync_grad(self.weight, self.bias)
        if x.is_cuda:
            from ...ops import norm_fused

            out = norm_fused.maybe_fused_layer_norm(x, w, b, self.col_group, self.eps)
            if out is not None:
                return out
        return distributed_layer_norm(x, w, b, self.col_group, self.eps)

    # ------------------------------------------------------------------ conversion
    @classmethod
    def convert_to_jigsaw(
        cls, model: torch.nn.LayerNorm, process_mesh_dict: dict, device: torch.device | str, row_kw: str = "row",
        col_kw: str = "col", model_kw: str = "model", **kwargs: Any,
    ) -> "DistributedLayerNorm":
        if len(model.normalized_shape) != 1:
            raise NotImplementedError("DistributedLayerNorm normalizes a single trailing dimension only")
        col = process_mesh_dict[col_kw]
        layer = cls(
            model.normalized_shape[0], None, device, process_mesh_dict[row_kw], col, eps=model.eps,
            elementwise_affine=model.elementwise_affine, bias=model.bias is not None,
            dtype=None if model.weight is None else model.weight.dtype,
        )
        layer._load_global(model.weight, model.bias)
        return layer

    def _load_global(self, weight: torch.Tensor | None, bias: torch.Tensor | None) -> None:
        parts = 1 if self.col_group is None else self.col_group.size()
        r = 0 if self.col_group is None else self.col_group.rank()
        n = self.normalized_dim // parts
        with torch.no_grad():
            if weight is not None and self.weight is not None:
                self.weight.data = weight.detach()[r * n : (r + 1) * n].clone().to(self.device)
            if bias is not None and self.bias is not None:
                self.bias.data = bias.detach()[r * n : (r + 1) * n].clone().to(self.device)

    def merge_weights(self, from_process_mesh: dict, row_kw: str = "row", col_kw: str = "col",
                      model_kw: str = "model") -> tuple[torch.Tensor | None, torch.Tensor | None]:
        """All-gather the slices over the column group (``row_kw`` and ``model_kw`` are accepted for a uniform
        signature: the parameters are not cut over them)."""
        g = from_process_mesh[col_kw]
        with torch.no_grad():
            w = None if self.weight is None else gather_dim(self.weight.detach(), g, 0)
            b = None if self.bias is None else gather_dim(self.bias.detach(), g, 0)
        return w, b

    def convert_to_torch(self, process_mesh_dict: dict, row_kw: str = "row", col_kw: str = "col", model_kw: str = "model") -> torch.nn.LayerNorm:
        w, b = self.merge_weights(process_mesh_dict, col_kw=col_kw)
        layer = torch.nn.LayerNorm(self.normalized_dim, eps=self.eps, elementwise_affine=self.elementwise_affine,
                                   bias=self.bias is not None, device=self.device)
        if w is not None:
            layer.weight.data = w
        if b is not None:
            layer.bias.data = b
        return layer

    def reshard_parameters(self, from_process_mesh: dict, to_process_mesh: dict, pm_row_key: str = "row",
                           pm_col_key: str = "col", pm_model_key: str = "model") -> None:
        new_col = to_process_mesh[pm_col_key]
        check_divisible(self.normalized_dim, new_col.size(), "normalized_dim")
        w, b = self.merge_weights(from_process_mesh, col_kw=pm_col_key)
        self.row_group, self.col_group = to_process_mesh[pm_row_key], new_col
        if self.weight is not None:
            self.weight = torch.nn.Parameter(torch.empty(0, device=self.device, dtype=w.dtype))
        if self.bias is not None:
            self.bias = torch.nn.Parameter(torch.empty(0, device=self.device, dtype=b.dtype))
        self._load_global(w, b)
        self._mark()

    def shard_spec(self) -> dict:
        """Which dimension of which parameter is cut over which group (sharded checkpoints)."""
        cut = () if self.col_group is None else ((0, self.col_group),)
        return {"weight": cut, "bias": cut}

    def get_parameter_count(self) -> int:
        if not self.elementwise_affine:
            return 0
        return self.normalized_dim * (2 if self.bias is not None else 1)

    def extra_repr(self) -> str:
        return (
            f"({self.normalized_dim},), eps={self.eps}, elementwise_affine={self.elementwise_affine}, "
            f"bias={self.bias is not None}, " + shard_repr(row=self.row_group, col=self.col_group)
        )
