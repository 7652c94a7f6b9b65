"""Softmax, log-softmax and arg-max along a dimension that is sharded over a process group.

Softmax over a sharded dimension needs two cross-rank reductions: the maximum (for
stability; constant for the gradient) and the sum of exponentials (which also carries
gradient, summed over the ranks in backward).  Under autocast the computation runs in
fp32.  Arg-max returns GLOBAL indices and breaks ties towards the lowest global index.

Reference parity: jigsaw/modules/activation/_functional.py:23-91 (softmax), :94-177
(log-softmax), :180-220 (argmax).
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ..._core.autocast import promote_to_fp32_under_autocast
from ..._core.collectives import all_reduce_max, all_reduce_min, all_reduce_sum


def _live(group: dist.ProcessGroup | None) -> bool:
    return group is not None and group.size() > 1


def _global_max(x: torch.Tensor, dim: int, group: dist.ProcessGroup | None) -> torch.Tensor:
    m = all_reduce_max(x.detach().amax(dim=dim, keepdim=True), group)
    # rows that are entirely -inf would give inf - inf
    return torch.where(torch.isfinite(m), m, torch.zeros_like(m))


def distributed_softmax(x: torch.Tensor, dim: int = -1, group: dist.ProcessGroup | None = None) -> torch.Tensor:
    """``softmax`` along ``dim`` whose extent is split over ``group`` (local shard in, local shard out)."""
    if not _live(group):
        return torch.softmax(x, dim=dim)
    if x.is_cuda:
        from ...ops import softmax_fused

        y = softmax_fused.maybe_fused_softmax(x, dim, group, log=False)      # statistics exchanged inside the kernel
        if y is not None:
            return y
    in_dtype = x.dtype
    (x,) = promote_to_fp32_under_autocast(x)
    e = torch.exp(x - _global_max(x, dim, group))
    s = all_reduce_sum(e.sum(dim=dim, keepdim=True), group)
    y = e / s
    return y if torch.is_autocast_enabled(x.device.type) else y.to(in_dtype)


def distributed_log_softmax(x: torch.Tensor, dim: int = -1, group: dist.ProcessGroup | None = None) -> torch.Tensor:
    """``log_softmax`` along ``dim`` whose extent is split over ``group``."""
    if not _live(group):
        return torch.log_softmax(x, dim=dim)
    if x.is_cuda:
        from ...ops import softmax_fused

        y = softmax_fused.maybe_fused_softmax(x, dim, group, log=True)
        if y is not None:
            return y
    in_dtype = x.dtype
    (x,) = promote_to_fp32_under_autocast(x)
    shifted = x - _global_max(x, dim, group)
    s = all_reduce_sum(torch.exp(shifted).sum(dim=dim, keepdim=True), group)
    y = shifted - torch.log(s)
    return y if torch.is_autocast_enabled(x.device.type) else y.to(in_dtype)


@torch.no_grad()
def distributed_argmax(x: torch.Tensor, dim: int, group: dist.ProcessGroup | None = None) -> torch.Tensor:
    """Global index of the maximum along the sharded ``dim``; ties go to the lowest index."""
    if not _live(group):
        return x.argmax(dim=dim)
    local_val, local_idx = x.max(dim=dim)
    # torch.max returns the first maximal index on CPU but not necessarily on CUDA: pin it
    is_max = x == local_val.unsqueeze(dim)
    ar = torch.arange(x.shape[dim], device=x.device).view([-1 if i == dim % x.dim() else 1 for i in range(x.dim())])
    local_idx = torch.where(is_max, ar, torch.full_like(ar, x.shape[dim])).amin(dim=dim)
    best = all_reduce_max(local_val, group)
    offset = group.rank() * x.shape[dim]
    sentinel = group.size() * x.shape[dim]
    cand = torch.where(local_val == best, local_idx + offset, torch.full_like(local_idx, sentinel))
    return all_reduce_min(cand, group)
