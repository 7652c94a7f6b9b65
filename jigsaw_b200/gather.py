"""Gather and average helpers for sharded tensors.

``gather_results`` reassembles a tensor whose last two dimensions are block-distributed
over a ``row`` x ``col`` grid (block ``(r, c)`` on model rank ``r * ncols + c``);
``gather_1d_results`` concatenates shards along one dimension.  Both are built on the
placement primitives, so they work on any mesh that has the named axes.

Reference parity: jigsaw/gather.py:17-53 (averaging), :57-141 (2-D gather), :145-213 (1-D).
"""

from __future__ import annotations

from collections.abc import Iterable, Mapping

import torch
import torch.distributed as dist

from ._core.placement import gather_dim

__all__ = [
    "average_weights",
    "average_weights_module",
    "gather_results",
    "gather_results_as_list",
    "gather_1d_results",
    "gather_1d_results_list",
]


def _avg_(t: torch.Tensor, group: dist.ProcessGroup) -> None:
    # gloo has no AVG reduction: sum then divide (bitwise the same for powers of two)
    if "gloo" in str(dist.get_backend(group)) and not t.is_cuda:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
        t.div_(group.size())
    else:
        dist.all_reduce(t, op=dist.ReduceOp.AVG, group=group)


@torch.no_grad()
def average_weights(params: Iterable[torch.Tensor | None], spatial_group: dist.ProcessGroup) -> None:
    """Average tensors in place over ``spatial_group`` (``None`` entries are skipped)."""
    for p in params:
        if p is not None:
            _avg_(p, spatial_group)


@torch.no_grad()
def average_weights_module(model: torch.nn.Module, spatial_group: dist.ProcessGroup, bias_only: bool = False) -> None:
    """Average every parameter of ``model`` (or only those named ``*bias*``) over ``spatial_group``."""
    for name, p in model.named_parameters():
        if bias_only and "bias" not in name:
            continue
        _avg_(p, spatial_group)


@torch.no_grad()
def gather_results(
    x: torch.Tensor,
    process_mesh_dict: Mapping[str, dist.ProcessGroup],
    pm_key_row: str = "row",
    pm_key_col: str = "col",
    pm_key_model: str = "model",
) -> torch.Tensor:
    """Full tensor from blocks of the last two dimensions (rows over ``pm_key_row``, columns
    over ``pm_key_col``).  ``pm_key_model`` is accepted for signature compatibility."""
    full = gather_dim(x, process_mesh_dict[pm_key_col], -1)
    return gather_dim(full, process_mesh_dict[pm_key_row], -2)


@torch.no_grad()
def gather_results_as_list(
    x: torch.Tensor,
    process_mesh: Mapping[str, dist.ProcessGroup] | None = None,
    pm_key_row: str = "row",
    pm_key_col: str = "col",
    pm_key_model: str = "model",
) -> list[torch.Tensor]:
    """The shard of every model rank, in model-rank order (``r * ncols + c``)."""
    if process_mesh is None:
        group = None
        n = dist.get_world_size()
    else:
        group = process_mesh[pm_key_model]
        n = group.size()
    x = x.contiguous()
    out = [torch.empty_like(x) for _ in range(n)]
    dist.all_gather(out, x, group=group)
    return out


@torch.no_grad()
def gather_1d_results(
    x: torch.Tensor, process_mesh_dict: Mapping[str, dist.ProcessGroup], dim: int = -1, pm_key: str = "model"
) -> torch.Tensor:
    """Concatenate the shards of ``process_mesh_dict[pm_key]`` along ``dim``."""
    return gather_dim(x, process_mesh_dict[pm_key], dim)


@torch.no_grad()
def gather_1d_results_list(
    x: torch.Tensor, process_mesh_dict: Mapping[str, dist.ProcessGroup], pm_key: str = "model"
) -> list[torch.Tensor]:
    """The shard of every rank of ``process_mesh_dict[pm_key]``, in group-rank order."""
    group = process_mesh_dict[pm_key]
    x = x.contiguous()
    out = [torch.empty_like(x) for _ in range(group.size())]
    dist.all_gather(out, x, group=group)
    return out
