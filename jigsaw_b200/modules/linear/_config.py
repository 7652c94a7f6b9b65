"""``LinearConfig``: transport and layout of a 2-D block-distributed matrix product.

Reference parity: jigsaw/modules/linear/_config.py:17-105.  The reference selects one of
four hand-written kernels per group size (1, 2, 4, 8 ranks = 1x1, 1x2, 2x2, 4x2 grids);
here one generic R x C schedule serves every grid, and the config records the grid.
"""

from __future__ import annotations

import copy

import torch
import torch.distributed as dist

from ..._core.comm import CommOp, resolve_comm_op

_GRIDS = {1: (1, 1), 2: (1, 2), 4: (2, 2), 8: (4, 2)}


def default_grid(model_size: int) -> tuple[int, int]:
    """Rows x columns of the block grid a bare model group of ``model_size`` ranks stands for."""
    if model_size not in _GRIDS:
        raise NotImplementedError(
            f"a model group of {model_size} ranks has no default block grid; supported sizes: {sorted(_GRIDS)}"
        )
    return _GRIDS[model_size]


class LinearConfig:
    """Kernel configuration of ``DistributedLinear`` and the ``DistributedMatMul*`` modules."""

    def __init__(
        self,
        model_group: dist.ProcessGroup | None,
        *,
        linear_layer: bool = True,
        device: torch.device | str = "cuda",
        comm: CommOp | str = "auto",
    ) -> None:
        self.device = torch.device(device)
        self.comm = resolve_comm_op(comm, self.device)
        self.linear_layer = linear_layer
        self.model_size = 1 if model_group is None else model_group.size()          # None: a single process
        self._layer_key = {"model group size": self.model_size, "linear_layer": linear_layer}
        self.vmapped = False

    def for_vmap(self) -> "LinearConfig":
        other = copy.copy(self)
        other.vmapped = True
        return other
