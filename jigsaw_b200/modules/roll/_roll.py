"""``torch.roll`` for tensors tiled over process groups.

A global cyclic shift by ``s`` along a dimension split into ``P`` tiles of ``n`` elements:
write ``s mod (P n) = q n + rem``.  Output tile ``r`` is the last ``rem`` elements of input
tile ``r - q - 1`` followed by the first ``n - rem`` elements of input tile ``r - q``.  Each
rank therefore sends two slabs (one of them possibly empty or local) around the ring; the
backward is the roll by ``-s`` and falls out of the differentiable ring pass.  Any shift
is supported (the reference requires ``|shift| <= local extent``).

On CUDA, contiguous bf16/fp32 inputs take the fused roll kernel of ``jigsaw_b200.ops``
that writes the wrapped slab straight into the neighbour's output buffer.

Reference parity: jigsaw/modules/roll/_roll.py:14-62 (Roll), :65-263 (DistributedRoll),
_distributed_roll.py:9-113, _functional.py:24-147, _config.py:8-27.
"""

from __future__ import annotations

from collections.abc import Sequence
from typing import Any

import torch
import torch.distributed as dist

from ..._core.collectives import ring_pass
from ..._core.comm import CommOp, resolve_comm_op
from ..._core.shard_repr import shard_repr


class RollConfig:
    """Transport of the slab exchange of :class:`DistributedRoll`."""

    def __init__(self, device: torch.device | str = "cuda", comm: CommOp | str = "auto") -> None:
        self.device = torch.device(device)
        self.comm = resolve_comm_op(comm, self.device)
        self._layer_key: dict = {}


def _tuple(x: int | Sequence[int]) -> tuple[int, ...]:
    return (x,) if isinstance(x, int) else tuple(x)


class Roll(torch.nn.Module):
    """``torch.roll`` as a module, convertible to :class:`DistributedRoll`."""

    def __init__(self, shifts: int | Sequence[int], dims: int | Sequence[int], dtype: torch.dtype = torch.float32) -> None:
        super().__init__()
        self.shifts, self.dims, self.dtype = _tuple(shifts), _tuple(dims), dtype
        if len(self.shifts) != len(self.dims):
            raise ValueError("shifts and dims must have the same length")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return torch.roll(x, self.shifts, self.dims)

    def get_parameter_count(self) -> int:
        return 0

    def extra_repr(self) -> str:
        return f"shifts={self.shifts}, dims={self.dims}"


def distributed_roll_1d(x: torch.Tensor, shift: int, dim: int, group: dist.ProcessGroup, comm: CommOp) -> torch.Tensor:
    """Roll ``x`` by ``shift`` along ``dim``, which is split over ``group`` in equal tiles."""
    P, n = group.size(), x.shape[dim]
    s = shift % (P * n)
    if s == 0:
        return x
    q, rem = divmod(s, n)
    head = x.narrow(dim, 0, n - rem)              # goes to rank r + q, lands at the end
    moved_head = ring_pass(head, group, q % P, comm) if q % P else head
    if rem == 0:
        return moved_head
    tail = x.narrow(dim, n - rem, rem)            # goes to rank r + q + 1, lands at the front
    moved_tail = ring_pass(tail, group, (q + 1) % P, comm) if (q + 1) % P else tail
    return torch.cat((moved_tail, moved_head), dim=dim)


class DistributedRoll(torch.nn.Module):
    """Roll over ``dims`` by ``shifts``; the dims listed in ``distributed_dims`` are tiled over
    the matching entry of ``spatial_groups`` (the others roll locally)."""

    def __init__(
        self,
        shifts: Sequence[int],
        dims: Sequence[int],
        distributed_dims: Sequence[int],
        spatial_groups: Sequence[dist.ProcessGroup],
        device: torch.device | str,
        dtype: torch.dtype = torch.float32,
        config: RollConfig | None = None,
    ) -> None:
        super().__init__()
        self.shifts, self.dims = _tuple(shifts), _tuple(dims)
        if len(self.shifts) != len(self.dims):
            raise ValueError("shifts and dims must have the same length")
        self.device, self.dtype = torch.device(device), dtype
        self.config = config or RollConfig(self.device)
        if len(_tuple(distributed_dims)) != len(tuple(spatial_groups)):
            raise ValueError("distributed_dims and spatial_groups must align: one process group (or None) per distributed dimension")
        self.reshard(distributed_dims, spatial_groups)

    def reshard(self, distributed_dims: Sequence[int], spatial_groups: Sequence[dist.ProcessGroup]) -> None:
        """Re-bind the module to other process groups."""
        distributed_dims, spatial_groups = _tuple(distributed_dims), tuple(spatial_groups)
        if len(distributed_dims) != len(spatial_groups):
            raise ValueError(f"distributed_dims and spatial_groups have mismatched lengths ({len(distributed_dims)} and {len(spatial_groups)})")
        stray = [d for d in distributed_dims if d not in self.dims]
        if stray:
            raise ValueError(f"every distributed dimension must appear in dims={self.dims}: a dimension that is not rolled "
                             f"needs no exchange (got {stray})")
        self.distributed_dims, self.spatial_groups = distributed_dims, spatial_groups

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        nd = x.dim()
        where = {d % nd: g for d, g in zip(self.distributed_dims, self.spatial_groups)}
        if x.is_cuda:
            from ...ops import roll_fused

            out = roll_fused.maybe_fused_roll(x, self.shifts, self.dims, where)
            if out is not None:
                return out
        for s, d in zip(self.shifts, self.dims):
            g = where.get(d % nd)
            if g is None or g.size() == 1:
                x = torch.roll(x, s, d)
            else:
                x = distributed_roll_1d(x, s, d % nd, g, self.config.comm)
        return x

    @classmethod
    def convert_to_jigsaw(
        cls, roll: Roll, process_mesh_dict: dict, device: torch.device | str, row_kw: str = "row", col_kw: str = "col",
        model_kw: str = "model", dim_to_mesh_axis: dict | None = None, **kwargs: Any,
    ) -> "DistributedRoll":
        mapping = {-2: row_kw} if dim_to_mesh_axis is None else dim_to_mesh_axis
        dims = tuple(mapping)
        groups = tuple(process_mesh_dict[a] for a in mapping.values())
        return cls(roll.shifts, roll.dims, dims, groups, device, roll.dtype)

    def convert_to_torch(self, *args: Any, **kwargs: Any) -> Roll:
        return Roll(self.shifts, self.dims, self.dtype)

    def get_parameter_count(self) -> int:
        return 0

    def extra_repr(self) -> str:
        return (
            f"shifts={self.shifts}, dims={self.dims}, distributed_dims={self.distributed_dims}, "
            + shard_repr(spatial=self.spatial_groups)
        )
