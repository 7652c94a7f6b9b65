"""Differentiable collectives: each forward collective carries its adjoint as backward.

With these, a distributed layer is written as a composition (gather -> local op ->
reduce) and autograd derives the distributed backward, instead of hand-writing a
backward schedule per layer and layout.

=====================  =============================  =============================
function               forward                        backward
=====================  =============================  =============================
all_gather_cat         all-gather, concat along dim   reduce-scatter (sum) along dim
reduce_scatter_sum     reduce-scatter (sum) along dim all-gather, concat along dim
all_reduce_sum         all-reduce (sum)               all-reduce (sum)
copy_to_group          identity                       all-reduce (sum)
reduce_from_group      all-reduce (sum)               identity
ring_pass              send to r+d, receive from r-d  send to r-d, receive from r+d
all_to_all_dims        split dim a, concat dim b      split dim b, concat dim a
=====================  =============================  =============================

Reference parity: the collective call sites of jigsaw/modules/convolution/_common/
channel_comm.py:137-172, spatial_split.py:54-72, jigsaw/modules/loss/_common.py:41-114 and
jigsaw/modules/attention/_functional/ulysses.py:19-63.
"""

from __future__ import annotations

from typing import Any

import torch
import torch.distributed as dist

from .comm import CommOp, ring_shift
from .vmap import to_front


def _live(group: dist.ProcessGroup | None) -> bool:
    return group is not None and group.size() > 1


def _gather_cat(x: torch.Tensor, group: dist.ProcessGroup, dim: int) -> torch.Tensor:
    x = x.contiguous()
    parts = [torch.empty_like(x) for _ in range(group.size())]
    dist.all_gather(parts, x, group=group)
    parts[group.rank()] = x
    return torch.cat(parts, dim=dim)


def _scatter_sum(x: torch.Tensor, group: dist.ProcessGroup, dim: int) -> torch.Tensor:
    n = group.size()
    chunks = [c.contiguous() for c in x.chunk(n, dim=dim)]
    out = torch.empty_like(chunks[0])
    if x.is_cuda:
        dist.reduce_scatter(out, chunks, op=dist.ReduceOp.SUM, group=group)
    else:
        # gloo has no reduce-scatter: all-reduce, keep own block
        full = x.contiguous().clone()
        dist.all_reduce(full, op=dist.ReduceOp.SUM, group=group)
        out = full.chunk(n, dim=dim)[group.rank()].contiguous()
    return out


def _batched_dim(x: torch.Tensor, bdim: int | None, dim: int) -> tuple[torch.Tensor, int]:
    """vmap helper: batch dimension to the front, ``dim`` (non-negative, of the unbatched tensor)
    shifted behind it."""
    if bdim is None:
        return x, dim
    return to_front(x, bdim), dim + 1


class _AllGatherCat(torch.autograd.Function):
    @staticmethod
    def forward(x: torch.Tensor, group: dist.ProcessGroup, dim: int) -> torch.Tensor:
        return _gather_cat(x, group, dim)

    @staticmethod
    def setup_context(ctx: Any, inputs: tuple, output: Any) -> None:
        _, ctx.group, ctx.dim = inputs

    @staticmethod
    def backward(ctx: Any, g: torch.Tensor) -> tuple:
        return _ReduceScatterSum.apply(g, ctx.group, ctx.dim), None, None

    @staticmethod
    def vmap(info: Any, in_dims: tuple, x: torch.Tensor, group: dist.ProcessGroup, dim: int) -> tuple:
        xb, d = _batched_dim(x, in_dims[0], dim)
        return _AllGatherCat.apply(xb, group, d), 0


class _ReduceScatterSum(torch.autograd.Function):
    @staticmethod
    def forward(x: torch.Tensor, group: dist.ProcessGroup, dim: int) -> torch.Tensor:
        return _scatter_sum(x, group, dim)

    @staticmethod
    def setup_context(ctx: Any, inputs: tuple, output: Any) -> None:
        _, ctx.group, ctx.dim = inputs

    @staticmethod
    def backward(ctx: Any, g: torch.Tensor) -> tuple:
        return _AllGatherCat.apply(g, ctx.group, ctx.dim), None, None

    @staticmethod
    def vmap(info: Any, in_dims: tuple, x: torch.Tensor, group: dist.ProcessGroup, dim: int) -> tuple:
        xb, d = _batched_dim(x, in_dims[0], dim)
        return _ReduceScatterSum.apply(xb, group, d), 0


class _AllReduce(torch.autograd.Function):
    """mode: 'both' (sum fwd, sum bwd), 'fwd' (sum fwd, identity bwd), 'bwd' (identity fwd, sum bwd)."""

    @staticmethod
    def forward(x: torch.Tensor, groups: tuple, mode: str) -> torch.Tensor:
        if mode == "bwd":
            return x.view_as(x)
        y = x.contiguous().clone()
        for g in groups:
            dist.all_reduce(y, op=dist.ReduceOp.SUM, group=g)
        return y

    @staticmethod
    def setup_context(ctx: Any, inputs: tuple, output: Any) -> None:
        _, ctx.groups, ctx.mode = inputs

    @staticmethod
    def backward(ctx: Any, g: torch.Tensor) -> tuple:
        if ctx.mode == "fwd":
            return g, None, None
        # the gradient of a sum over ranks is again a sum over ranks (and differentiable in turn)
        return _AllReduce.apply(g, ctx.groups, "both"), None, None

    @staticmethod
    def vmap(info: Any, in_dims: tuple, x: torch.Tensor, groups: tuple, mode: str) -> tuple:
        return _AllReduce.apply(x, groups, mode), in_dims[0]


class _RingPass(torch.autograd.Function):
    @staticmethod
    def forward(x: torch.Tensor, group: dist.ProcessGroup, direction: int, comm: CommOp) -> torch.Tensor:
        out, _ = ring_shift(x.contiguous(), None, direction, group, comm)
        return out

    @staticmethod
    def setup_context(ctx: Any, inputs: tuple, output: Any) -> None:
        _, ctx.group, ctx.direction, ctx.comm = inputs

    @staticmethod
    def backward(ctx: Any, g: torch.Tensor) -> tuple:
        return _RingPass.apply(g, ctx.group, -ctx.direction, ctx.comm), None, None, None

    @staticmethod
    def vmap(info: Any, in_dims: tuple, x: torch.Tensor, group: dist.ProcessGroup, direction: int, comm: CommOp) -> tuple:
        return _RingPass.apply(x, group, direction, comm), in_dims[0]      # whole tensors travel: any layout


def _a2a(x: torch.Tensor, group: dist.ProcessGroup, split_dim: int, cat_dim: int) -> torch.Tensor:
    if x.is_cuda:
        from ..ops import exchange_fused

        out = exchange_fused.maybe_fused_all_to_all(x, group, split_dim, cat_dim)     # one kernel over peer memory
        if out is not None:
            return out
    n = group.size()
    ins = [c.contiguous() for c in x.chunk(n, dim=split_dim)]
    outs = [torch.empty_like(ins[0]) for _ in range(n)]
    if x.is_cuda:
        dist.all_to_all(outs, ins, group=group)
    else:
        from .comm import sparse_exchange

        sparse_exchange(dict(enumerate(ins)), dict(enumerate(outs)), group, CommOp.BATCH_ISEND_IRECV)
    return torch.cat(outs, dim=cat_dim)


class _AllToAllDims(torch.autograd.Function):
    @staticmethod
    def forward(x: torch.Tensor, group: dist.ProcessGroup, split_dim: int, cat_dim: int) -> torch.Tensor:
        return _a2a(x, group, split_dim, cat_dim)

    @staticmethod
    def setup_context(ctx: Any, inputs: tuple, output: Any) -> None:
        _, ctx.group, ctx.split_dim, ctx.cat_dim = inputs

    @staticmethod
    def backward(ctx: Any, g: torch.Tensor) -> tuple:
        return _AllToAllDims.apply(g, ctx.group, ctx.cat_dim, ctx.split_dim), None, None, None

    @staticmethod
    def vmap(info: Any, in_dims: tuple, x: torch.Tensor, group: dist.ProcessGroup, split_dim: int, cat_dim: int) -> tuple:
        if in_dims[0] is None:
            return _AllToAllDims.apply(x, group, split_dim, cat_dim), None
        return _AllToAllDims.apply(x.movedim(in_dims[0], 0), group, split_dim + 1, cat_dim + 1), 0


class _ReduceNoGrad(torch.autograd.Function):
    """Element-wise MAX / MIN all-reduce of a detached tensor (no gradient flows); elementwise in
    every dimension, so ``vmap`` passes the batch dimension straight through."""

    @staticmethod
    def forward(x: torch.Tensor, group: dist.ProcessGroup, op: Any) -> torch.Tensor:
        y = x.detach().contiguous().clone()
        dist.all_reduce(y, op=op, group=group)
        return y

    @staticmethod
    def setup_context(ctx: Any, inputs: tuple, output: Any) -> None:
        ctx.mark_non_differentiable(output)

    @staticmethod
    def backward(ctx: Any, g: torch.Tensor) -> tuple:
        return None, None, None

    @staticmethod
    def vmap(info: Any, in_dims: tuple, x: torch.Tensor, group: dist.ProcessGroup, op: Any) -> tuple:
        return _ReduceNoGrad.apply(x, group, op), in_dims[0]


def all_reduce_max(x: torch.Tensor, group: dist.ProcessGroup | None) -> torch.Tensor:
    """Element-wise maximum over the group (detached)."""
    return _ReduceNoGrad.apply(x, group, dist.ReduceOp.MAX) if _live(group) else x.detach()


def all_reduce_min(x: torch.Tensor, group: dist.ProcessGroup | None) -> torch.Tensor:
    """Element-wise minimum over the group (detached)."""
    return _ReduceNoGrad.apply(x, group, dist.ReduceOp.MIN) if _live(group) else x.detach()


def _norm_groups(groups: Any) -> tuple:
    if groups is None:
        return ()
    if isinstance(groups, dist.ProcessGroup):
        groups = (groups,)
    gs = tuple(g for g in groups if _live(g))
    if len(gs) > 1:
        # axes that tile a whole model replica: one collective over the flattened group
        from ..parallel._replicas import merged_group

        whole = merged_group(gs)
        if whole is not None:
            return (whole,)
    return gs


def all_gather_cat(x: torch.Tensor, group: dist.ProcessGroup | None, dim: int) -> torch.Tensor:
    """Concatenate every rank's ``x`` along ``dim``; gradient is reduce-scattered back."""
    if not _live(group):
        return x
    return _AllGatherCat.apply(x, group, dim % x.dim())


def reduce_scatter_sum(x: torch.Tensor, group: dist.ProcessGroup | None, dim: int) -> torch.Tensor:
    """Sum over the group and keep this rank's block of ``dim``; gradient is all-gathered."""
    if not _live(group):
        return x
    return _ReduceScatterSum.apply(x, group, dim % x.dim())


def all_reduce_sum(x: torch.Tensor, groups: Any) -> torch.Tensor:
    """Sum over ``groups`` in forward and in backward."""
    gs = _norm_groups(groups)
    return _AllReduce.apply(x, gs, "both") if gs else x


def reduce_from_group(x: torch.Tensor, groups: Any) -> torch.Tensor:
    """Sum over ``groups`` in forward; identity gradient (every rank already holds the full
    upstream gradient of the replicated result)."""
    gs = _norm_groups(groups)
    return _AllReduce.apply(x, gs, "fwd") if gs else x


def copy_to_group(x: torch.Tensor, groups: Any) -> torch.Tensor:
    """Identity in forward; gradient summed over ``groups`` (a replicated value consumed by
    rank-local computations)."""
    gs = _norm_groups(groups)
    return _AllReduce.apply(x, gs, "bwd") if gs else x


def ring_pass(x: torch.Tensor, group: dist.ProcessGroup | None, direction: int, comm: CommOp) -> torch.Tensor:
    """Cyclic shift by ``direction`` ranks; the gradient travels the other way."""
    if not _live(group):
        return x
    return _RingPass.apply(x, group, direction, comm)


def all_to_all_dims(x: torch.Tensor, group: dist.ProcessGroup | None, split_dim: int, cat_dim: int) -> torch.Tensor:
    """Re-shard: split ``split_dim`` over the group, concatenate what arrives along ``cat_dim``."""
    if not _live(group):
        return x
    return _AllToAllDims.apply(x, group, split_dim % x.dim(), cat_dim % x.dim())
