"""``DistributedSoftmax`` module.

Reference parity: jigsaw/modules/activation/_activation.py:13-125.
"""

from __future__ import annotations

from typing import Any

import torch
import torch.distributed as dist

from ..._core.shard_repr import shard_repr
from ._functional import distributed_softmax


class DistributedSoftmax(torch.nn.Module):
    """Softmax along ``dim`` whose extent is split over ``group``."""

    def __init__(self, group: dist.ProcessGroup | None, dim: int = -1) -> None:
        super().__init__()
        self.group = group
        self.dim = dim

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return distributed_softmax(x, self.dim, self.group)

    @classmethod
    def convert_to_jigsaw(
        cls, model: torch.nn.Softmax, process_mesh_dict: dict, device: Any = None, row_kw: str = "row",
        col_kw: str = "col", model_kw: str = "model", **kwargs: Any,
    ) -> "DistributedSoftmax":
        """The softmax dimension is taken to be the feature dimension, split over ``col_kw``.  A ``Softmax`` built
        without ``dim`` picks its axis from the rank of each input (torch's legacy rule), which a layer that must
        know whether its axis is cut cannot follow: that one is refused."""
        if model.dim is None:
            raise NotImplementedError("a Softmax without an explicit dim cannot be converted: give it the dim it normalises, "
                                      "or build DistributedSoftmax(group, dim) by hand")
        return cls(kwargs.get("group", process_mesh_dict[col_kw]), model.dim)

    def convert_to_torch(self, *args: Any, **kwargs: Any) -> torch.nn.Softmax:
        return torch.nn.Softmax(dim=self.dim)

    def get_parameter_count(self) -> int:
        return 0

    def extra_repr(self) -> str:
        return f"dim={self.dim}, " + shard_repr(group=self.group)
