"""Gradient clipping by the norm of the whole (unsharded) model's gradient.

Each rank holds shards of some parameters and full copies of others.  The global p-norm
counts every element once: a shard contributes its local norm^p, a parameter replicated
over groups ``R`` contributes norm^p / prod(|g| for g in R).  Accumulation is float64;
the infinity norm needs a MAX instead and no correction.

Reference parity: jigsaw/parallel/_clip.py:13-111 (clip), :114-179 (norm helpers, copy count).
"""

from __future__ import annotations

import math
from collections.abc import Iterable

import torch
import torch.distributed as dist

from .._core.comm import get_device_of_process_group
from ._replicas import Groups, replica_groups


def _copy_count(groups: Groups, clip_group: dist.ProcessGroup, cache: dict[Groups, int]) -> int:
    if groups in cache:
        return cache[groups]
    if groups:
        inside = set(dist.get_process_group_ranks(clip_group))
        for g in groups:
            ranks = dist.get_process_group_ranks(g)
            if not inside.issuperset(ranks):
                raise ValueError(
                    f"a parameter is replicated over ranks {ranks}, not all in the clipping group "
                    f'{sorted(inside)}; pass the model-parallel group, e.g. mesh["model"].'
                )
    cache[groups] = math.prod(g.size() for g in groups)
    return cache[groups]


def _local_norms(grads: list[torch.Tensor], p: float, device: torch.device) -> torch.Tensor:
    """Per-gradient norms as one float64 vector (each accumulated in >= float32)."""
    by_kind: dict[tuple[torch.device, torch.dtype], list[torch.Tensor]] = {}
    for g in grads:
        by_kind.setdefault((g.device, g.dtype), []).append(g)
    parts = []
    for (_, dt), gs in by_kind.items():
        acc = torch.promote_types(dt, torch.float32)
        parts.append(torch.stack(torch._foreach_norm(gs, p, dtype=acc)).to(device, torch.float64))
    return torch.cat(parts)


def clip_grad_norm_(
    parameters: torch.Tensor | Iterable[torch.Tensor],
    max_norm: float,
    group: dist.ProcessGroup,
    norm_type: float = 2.0,
    error_if_nonfinite: bool = False,
) -> torch.Tensor:
    """Same result as ``torch.nn.utils.clip_grad_norm_`` on the unsharded model.

    Collective over ``group`` (the model-parallel group): call on every rank after
    backward, also on ranks without gradients.  Returns the total norm before clipping in
    the promoted dtype of the parameters (at least float32).
    """
    if isinstance(parameters, torch.Tensor):
        parameters = [parameters]
    p = float(norm_type)
    dtype = torch.float32
    cache: dict[Groups, int] = {}
    by_copies: dict[int, list[torch.Tensor]] = {}
    grads: list[torch.Tensor] = []
    for param in parameters:  # visit all, so every rank agrees on dtype and raises together
        dtype = torch.promote_types(dtype, param.dtype)
        n = _copy_count(replica_groups(param), group, cache)
        if param.grad is not None:
            grads.append(param.grad)
            by_copies.setdefault(n, []).append(param.grad)
    device = grads[0].device if grads else get_device_of_process_group(group)
    with torch.no_grad():
        total = torch.zeros((), dtype=torch.float64, device=device)
        if math.isinf(p):
            if grads:
                total = _local_norms(grads, p, device).max()
            dist.all_reduce(total, op=dist.ReduceOp.MAX, group=group)
        else:
            for n, gs in by_copies.items():
                total = total + _local_norms(gs, p, device).pow(p).sum() / n
            dist.all_reduce(total, op=dist.ReduceOp.SUM, group=group)
            total = total.pow(1.0 / p)
        if error_if_nonfinite and not bool(torch.isfinite(total)):
            raise RuntimeError(
                f"The total norm of order {p} for gradients from `parameters` is non-finite, so it "
                "cannot be clipped. To disable this error and scale the gradients by the non-finite "
                "norm anyway, set `error_if_nonfinite=False`"
            )
        coef = torch.clamp(max_norm / (total + 1e-6), max=1.0)
        by_kind: dict[tuple[torch.device, torch.dtype], list[torch.Tensor]] = {}
        for g in grads:
            by_kind.setdefault((g.device, g.dtype), []).append(g)
        for (dev, dt), gs in by_kind.items():
            torch._foreach_mul_(gs, coef.to(dev, dt))
    return total.to(dtype)
