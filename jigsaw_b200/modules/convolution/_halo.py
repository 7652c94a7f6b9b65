"""Span exchange along one split axis: the halo gather of a convolution and its adjoint.

Along a split axis every rank *owns* the range ``[r * own, (r + 1) * own)`` of a global
axis and *holds* a span ``[lo_r, lo_r + held)`` of it that may reach into neighbours (and
beyond the global domain, where values are zero):

* ``span_gather`` : owned block -> held span (copy from the owners; zero outside).  It is
  the input halo gather of a convolution and the gradient expansion of a transposed one.
* ``span_reduce`` : held span -> owned block (contributions are summed on their owner,
  positions outside the domain dropped).  It is the output halo reduce of a transposed
  convolution and the gradient scatter-add of a convolution.

The two are adjoint, so each is the other's backward.  Spans of every rank follow from
closed-form arithmetic, so no metadata is communicated; spans wider than one neighbour
(large kernels or dilations on small tiles) simply intersect more owners.

Reference parity: jigsaw/modules/convolution/_conv/halo.py:9-63 (needed_input_span),
:66-156 (halo_gather), :159-251 (halo_scatter_add); _conv_transpose/halo.py:55-69
(produced span), :72-162 (transpose_halo_reduce), :165-258 (transpose_halo_expand);
_common/halo.py:7-63 (exchange_along_axis).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch
import torch.distributed as dist

from ..._core.comm import CommOp, sparse_exchange


class UnevenSplitError(NotImplementedError, ValueError):
    """The output of a layer does not divide evenly over the ranks of a split axis.  A ``NotImplementedError``
    (uneven tiles are not supported; the reference raises that type) which is also a ``ValueError`` (the sizes
    passed in are what is wrong)."""


@dataclass(frozen=True)
class AxisPlan:
    """Geometry of one split axis.  ``lo[q]`` is the global start of rank ``q``'s held span."""

    dim: int                   # tensor dimension (negative, counted from the end)
    group: dist.ProcessGroup
    own: int                   # owned extent per rank
    held: int                  # held extent per rank
    lo: tuple[int, ...]        # held-span start per group rank (global coordinates)
    comm: CommOp

    @property
    def total(self) -> int:
        return self.own * len(self.lo)

    def overlap(self, holder: int, owner: int) -> tuple[int, int]:
        """Global ``[a, b)`` of what ``holder`` holds from the range owned by ``owner``."""
        a = max(self.lo[holder], owner * self.own, 0)
        b = min(self.lo[holder] + self.held, (owner + 1) * self.own, self.total)
        return a, max(a, b)


def conv_axis_plan(
    dim: int, group: dist.ProcessGroup, n_local: int, kernel: int, stride: int, padding: int, dilation: int, comm: CommOp
) -> tuple[AxisPlan, int]:
    """Input span each rank needs for its share of the convolution output.

    Returns the plan and the local output extent.  Raises ``ValueError`` when the global
    output does not divide evenly over the group.
    """
    G = group.size()
    extent = dilation * (kernel - 1) + 1
    global_out = (G * n_local + 2 * padding - extent) // stride + 1
    if global_out <= 0 or global_out % G != 0:
        raise UnevenSplitError(
            f"global output size {global_out} along a split axis must be positive and divisible by the "
            f"spatial group size {G} (local input {n_local}, kernel {kernel}, stride {stride}, "
            f"padding {padding}, dilation {dilation})"
        )
    out_local = global_out // G
    held = (out_local - 1) * stride + extent
    lo = tuple(q * out_local * stride - padding for q in range(G))
    return AxisPlan(dim, group, n_local, held, lo, comm), out_local


def conv_transpose_axis_plan(
    dim: int, group: dist.ProcessGroup, n_local: int, kernel: int, stride: int, padding: int, dilation: int, comm: CommOp
) -> AxisPlan:
    """Output span each rank produces (raw local transposed convolution, padding 0 on the axis)."""
    G = group.size()
    extent = dilation * (kernel - 1) + 1
    global_out = (G * n_local - 1) * stride - 2 * padding + extent
    if global_out <= 0 or global_out % G != 0:
        raise UnevenSplitError(
            f"global output size {global_out} along a split axis must be positive and divisible by the "
            f"spatial group size {G} (local input {n_local}, kernel {kernel}, stride {stride}, padding {padding})"
        )
    out_local = global_out // G
    held = (n_local - 1) * stride + extent
    lo = tuple(q * n_local * stride - padding for q in range(G))
    return AxisPlan(dim, group, out_local, held, lo, comm)


def _gather(x: torch.Tensor, plan: AxisPlan) -> torch.Tensor:
    me, G = plan.group.rank(), plan.group.size()
    dim = plan.dim % x.dim()
    shape = list(x.shape)
    shape[dim] = plan.held
    out = x.new_empty(shape)
    # the owners' ranges tile the domain without gaps, so the held span is covered except where it reaches
    # beyond the domain: only those two ends are zero-filled (no pass over the whole buffer)
    lo, hi = plan.lo[me], plan.lo[me] + plan.held
    below, above = min(max(0, lo), hi) - lo, hi - max(min(plan.total, hi), lo)
    if below > 0:
        out.narrow(dim, 0, below).zero_()
    if above > 0:
        out.narrow(dim, plan.held - above, above).zero_()
    sends: dict[int, torch.Tensor] = {}
    recvs: dict[int, torch.Tensor] = {}
    landing: list[tuple[int, int, torch.Tensor]] = []
    for q in range(G):
        a, b = plan.overlap(me, q)          # what I hold from q
        if b > a:
            if q == me:
                out.narrow(dim, a - plan.lo[me], b - a).copy_(x.narrow(dim, a - me * plan.own, b - a))
            else:
                rshape = list(x.shape)
                rshape[dim] = b - a
                buf = x.new_empty(rshape)
                recvs[q] = buf
                landing.append((a - plan.lo[me], b - a, buf))
        if q != me:
            a, b = plan.overlap(q, me)      # what q holds from me
            if b > a:
                sends[q] = x.narrow(dim, a - me * plan.own, b - a).contiguous()
    sparse_exchange(sends, recvs, plan.group, plan.comm)
    for start, length, buf in landing:
        out.narrow(dim, start, length).copy_(buf)
    return out


def _reduce(y: torch.Tensor, plan: AxisPlan) -> torch.Tensor:
    me, G = plan.group.rank(), plan.group.size()
    dim = plan.dim % y.dim()
    shape = list(y.shape)
    shape[dim] = plan.own
    a, b = plan.overlap(me, me)
    covers = b - a == plan.own              # my held span contains everything I own: start from that piece, not from zeros
    out = y.narrow(dim, a - plan.lo[me], b - a).clone(memory_format=torch.contiguous_format) if covers else y.new_zeros(shape)
    sends: dict[int, torch.Tensor] = {}
    recvs: dict[int, torch.Tensor] = {}
    landing: list[tuple[int, int, torch.Tensor]] = []
    for q in range(G):
        a, b = plan.overlap(me, q)          # part of my held span owned by q
        if b > a:
            piece = y.narrow(dim, a - plan.lo[me], b - a)
            if q == me:
                if not covers:
                    out.narrow(dim, a - me * plan.own, b - a).add_(piece)
            else:
                sends[q] = piece.contiguous()
        if q != me:
            a, b = plan.overlap(q, me)      # part of q's held span that I own
            if b > a:
                rshape = list(y.shape)
                rshape[dim] = b - a
                buf = y.new_empty(rshape)
                recvs[q] = buf
                landing.append((a - me * plan.own, b - a, buf))
    sparse_exchange(sends, recvs, plan.group, plan.comm)
    for start, length, buf in landing:
        out.narrow(dim, start, length).add_(buf)
    return out


class _SpanGather(torch.autograd.Function):
    @staticmethod
    def forward(x: torch.Tensor, plan: AxisPlan) -> torch.Tensor:
        return _gather(x, plan)

    @staticmethod
    def setup_context(ctx: Any, inputs: tuple, output: Any) -> None:
        ctx.plan = inputs[1]

    @staticmethod
    def backward(ctx: Any, g: torch.Tensor) -> tuple:
        return _SpanReduce.apply(g, ctx.plan), None

    @staticmethod
    def vmap(info: Any, in_dims: tuple, x: torch.Tensor, plan: AxisPlan) -> tuple:
        # the plan addresses its axis from the end, so a leading batch dimension does not disturb it
        if in_dims[0] is None:
            return _SpanGather.apply(x, plan), None
        return _SpanGather.apply(x.movedim(in_dims[0], 0), plan), 0


class _SpanReduce(torch.autograd.Function):
    @staticmethod
    def forward(y: torch.Tensor, plan: AxisPlan) -> torch.Tensor:
        return _reduce(y, plan)

    @staticmethod
    def setup_context(ctx: Any, inputs: tuple, output: Any) -> None:
        ctx.plan = inputs[1]

    @staticmethod
    def backward(ctx: Any, g: torch.Tensor) -> tuple:
        return _SpanGather.apply(g, ctx.plan), None

    @staticmethod
    def vmap(info: Any, in_dims: tuple, y: torch.Tensor, plan: AxisPlan) -> tuple:
        if in_dims[0] is None:
            return _SpanReduce.apply(y, plan), None
        return _SpanReduce.apply(y.movedim(in_dims[0], 0), plan), 0


def span_gather(x: torch.Tensor, plan: AxisPlan) -> torch.Tensor:
    """Owned block -> held span (differentiable; backward is :func:`span_reduce`)."""
    return _SpanGather.apply(x, plan)


def span_reduce(y: torch.Tensor, plan: AxisPlan) -> torch.Tensor:
    """Held span -> owned block, summing overlaps (differentiable; backward is :func:`span_gather`)."""
    return _SpanReduce.apply(y, plan)
