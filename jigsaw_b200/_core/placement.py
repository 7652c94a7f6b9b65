"""Placement model: how a tensor is laid out over process groups.

A placement is a list of ``(group, dim)`` pairs: the tensor is split in equal blocks along
``dim`` over ``group`` (block index = group rank).  Anything not listed is replicated.
Sharding, gathering, resharding, parameter counting and checkpoint manifests are all
expressed through these few functions instead of per-layout rank tables.

Reference parity: the layout knowledge spread over jigsaw/gather.py:57-213 and the
``merge_weights`` / ``reshard_parameters`` methods of every layer
(jigsaw/modules/linear/_linear.py:433-594 and siblings).
"""

from __future__ import annotations

from collections.abc import Sequence
from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class Shard:
    """Equal split of dimension ``dim`` over ``group``."""

    group: dist.ProcessGroup | None
    dim: int

    @property
    def parts(self) -> int:
        return 1 if self.group is None else self.group.size()

    @property
    def index(self) -> int:
        return 0 if self.group is None else self.group.rank()


def shard_dim(x: torch.Tensor, group: dist.ProcessGroup | None, dim: int, *, what: str = "tensor") -> torch.Tensor:
    """This rank's block of ``x`` along ``dim`` (a view; clone before owning it)."""
    if group is None or group.size() == 1:
        return x
    n = group.size()
    if x.shape[dim] % n != 0:
        raise ValueError(f"{what}: dimension {dim} of size {x.shape[dim]} is not divisible by {n} ranks")
    block = x.shape[dim] // n
    return x.narrow(dim, group.rank() * block, block)


def gather_dim(x: torch.Tensor, group: dist.ProcessGroup | None, dim: int) -> torch.Tensor:
    """Concatenate the blocks of every rank of ``group`` along ``dim`` (collective)."""
    if group is None or group.size() == 1:
        return x
    x = x.contiguous()
    parts = [torch.empty_like(x) for _ in range(group.size())]
    dist.all_gather(parts, x, group=group)
    return torch.cat(parts, dim=dim)


def shard(x: torch.Tensor, placement: Sequence[Shard], *, what: str = "tensor") -> torch.Tensor:
    """Apply every split of ``placement`` in order and return an owned, contiguous block."""
    for s in placement:
        x = shard_dim(x, s.group, s.dim, what=what)
    return x.contiguous().clone() if placement else x


def gather(x: torch.Tensor, placement: Sequence[Shard]) -> torch.Tensor:
    """Inverse of :func:`shard` (collective over every group of the placement)."""
    for s in reversed(list(placement)):
        x = gather_dim(x, s.group, s.dim)
    return x


def global_shape(local_shape: Sequence[int], placement: Sequence[Shard]) -> tuple[int, ...]:
    shape = list(local_shape)
    for s in placement:
        shape[s.dim] *= s.parts
    return tuple(shape)


def check_divisible(value: int, parts: int, what: str) -> int:
    """Return ``value // parts`` or raise ``ValueError`` naming ``what``."""
    if parts < 1 or value % parts != 0:
        raise ValueError(f"{what}={value} must be divisible by the group size {parts}")
    return value // parts
