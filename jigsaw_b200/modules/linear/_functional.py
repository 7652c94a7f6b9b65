"""2-D block-distributed matrix products as compositions of differentiable collectives.

Grid R x C, rank ``(i, j) = i * C + j`` of the model group.  Every operand and result is
block-distributed over its LAST TWO dimensions exactly as ``gather_results`` reassembles
them; leading dimensions are batch.

    XWT : Y = X  W^T   X (M/R, K/C)   W (N/R, K/C)   ->  Y (M/R, N/C)
    XW  : Y = X  W     X (M/R, K/C)   W (K/R, N/C)   ->  Y (M/R, N/C)
    XTW : Y = X^T W    X (K/R, M/C)   W (K/R, N/C)   ->  Y (M/R, N/C)

Schedule: fetch -> GEMM.  A rank fetches exactly the region of each operand that its result block
needs (for ``Y_ij`` of XWT: row block ``i`` of ``X`` over all of ``K`` and the ``N / C`` rows of ``W`` that
make output block ``j``), block by block from the ranks that own them, in one sparse exchange over the
model group (:func:`fetch_region`); nothing else is ever materialised, so the transient memory is the size
of the regions, not of the whole matrices.  The local product is one GEMM; the backward sends every
region's gradient back to the owners of its blocks, where the contributions of all readers are summed.

Reference parity: the 2/4/8-way kernels of jigsaw/modules/linear/_distributed_matmul.py
(:116-179 1x2, :294-413 2x2, :862-1181 4x2, :44-113 / :540-734 / :1843-2580 fused
backward) and their p2p variants; semantics pinned by
tests/modules/linear/test_matmul_nway.py:96-185.
"""

from __future__ import annotations

from typing import Any

import torch
import torch.distributed as dist

from ..._core.autocast import cast_to_autocast_dtype
from ..._core.comm import CommOp, resolve_comm_op, sparse_exchange
from ..._core.vmap import to_front

Region = tuple[int, int, int, int]          # rows [r0, r1) and columns [c0, c1) of the global matrix


def _overlap(a: Region, b: Region) -> Region | None:
    r0, r1, c0, c1 = max(a[0], b[0]), min(a[1], b[1]), max(a[2], b[2]), min(a[3], b[3])
    return (r0, r1, c0, c1) if r0 < r1 and c0 < c1 else None


def _transport(comm: CommOp | str, device: torch.device) -> CommOp:
    try:
        return resolve_comm_op(comm, device)
    except ValueError:                      # a transport chosen for another device type
        return resolve_comm_op("auto", device)


def _plan(h: int, w: int, group: dist.ProcessGroup, R: int, C: int, region_of: Any) -> tuple:
    """Who reads what: ``(mine, want, plan_send, plan_recv)`` for a local block of ``h x w`` elements.
    ``plan_send[p]`` is the part of my block that rank ``p`` reads, ``plan_recv[p]`` the part of rank
    ``p``'s block that I read (both in global coordinates)."""
    me = group.rank()
    block = lambda p: ((p // C) * h, (p // C + 1) * h, (p % C) * w, (p % C + 1) * w)  # noqa: E731
    mine, want = block(me), region_of(me)
    plan_send, plan_recv = {}, {}
    for p in range(R * C):
        give = _overlap(region_of(p), mine)
        if give is not None:
            plan_send[p] = give
        take = _overlap(want, block(p))
        if take is not None:
            plan_recv[p] = take
    return mine, want, plan_send, plan_recv


def _cut(t: torch.Tensor, part: Region, origin: Region) -> torch.Tensor:
    return t[..., part[0] - origin[0]:part[1] - origin[0], part[2] - origin[2]:part[3] - origin[2]]


def _fetch(x: torch.Tensor, group: dist.ProcessGroup, R: int, C: int, region_of: Any, comm: Any) -> torch.Tensor:
    x = x.contiguous()
    mine, want, plan_send, plan_recv = _plan(x.shape[-2], x.shape[-1], group, R, C, region_of)
    lead = x.shape[:-2]
    out = x.new_empty(*lead, want[1] - want[0], want[3] - want[2])
    sends = {p: _cut(x, give, mine).contiguous() for p, give in plan_send.items()}
    recvs = {p: x.new_empty(*lead, take[1] - take[0], take[3] - take[2]) for p, take in plan_recv.items()}
    sparse_exchange(sends, recvs, group, _transport(comm, x.device))
    for p, take in plan_recv.items():
        _cut(out, take, want).copy_(recvs[p])
    return out


def _scatter_add(g: torch.Tensor, h: int, w: int, group: dist.ProcessGroup, R: int, C: int, region_of: Any, comm: Any) -> torch.Tensor:
    """Adjoint of :func:`_fetch`: every piece of the region's gradient goes back to the owner of its
    block, where the contributions of all readers are summed (in fp32 at least)."""
    g = g.contiguous()
    mine, want, plan_send, plan_recv = _plan(h, w, group, R, C, region_of)
    lead = g.shape[:-2]
    sends = {p: _cut(g, take, want).contiguous() for p, take in plan_recv.items()}
    recvs = {p: g.new_empty(*lead, give[1] - give[0], give[3] - give[2]) for p, give in plan_send.items()}
    sparse_exchange(sends, recvs, group, _transport(comm, g.device))
    acc = torch.zeros(*lead, h, w, dtype=torch.promote_types(g.dtype, torch.float32), device=g.device)
    for p, give in plan_send.items():
        _cut(acc, give, mine).add_(recvs[p])
    return acc.to(g.dtype)


class _FetchRegion(torch.autograd.Function):
    """``region_of(rank)`` of a matrix whose last two dimensions are cut into ``R x C`` blocks over
    ``group`` (rank ``i * C + j`` holds block ``(i, j)``): every rank receives its region piece by piece
    from the owners of the blocks it overlaps.  Backward: the adjoint scatter-add (:class:`_ScatterRegion`),
    itself differentiable; leading dimensions are batch, which is also the ``vmap`` rule."""

    @staticmethod
    def forward(x: torch.Tensor, group: dist.ProcessGroup, R: int, C: int, region_of: Any, comm: Any) -> torch.Tensor:
        return _fetch(x, group, R, C, region_of, comm)

    @staticmethod
    def setup_context(ctx: Any, inputs: tuple, output: Any) -> None:
        x, ctx.group, ctx.R, ctx.C, ctx.region_of, ctx.comm = inputs
        ctx.hw, ctx.x_dtype = (x.shape[-2], x.shape[-1]), x.dtype

    @staticmethod
    def backward(ctx: Any, g: torch.Tensor) -> tuple:
        gx = _ScatterRegion.apply(g, ctx.hw[0], ctx.hw[1], ctx.group, ctx.R, ctx.C, ctx.region_of, ctx.comm)
        return gx.to(ctx.x_dtype), None, None, None, None, None

    @staticmethod
    def vmap(info: Any, in_dims: tuple, x: torch.Tensor, group: Any, R: int, C: int, region_of: Any, comm: Any) -> tuple:
        xb = to_front(x, in_dims[0])
        return _FetchRegion.apply(xb, group, R, C, region_of, comm), (None if in_dims[0] is None else 0)


class _ScatterRegion(torch.autograd.Function):
    @staticmethod
    def forward(g: torch.Tensor, h: int, w: int, group: dist.ProcessGroup, R: int, C: int, region_of: Any, comm: Any) -> torch.Tensor:
        return _scatter_add(g, h, w, group, R, C, region_of, comm)

    @staticmethod
    def setup_context(ctx: Any, inputs: tuple, output: Any) -> None:
        _, _, _, ctx.group, ctx.R, ctx.C, ctx.region_of, ctx.comm = inputs

    @staticmethod
    def backward(ctx: Any, gg: torch.Tensor) -> tuple:
        return _FetchRegion.apply(gg, ctx.group, ctx.R, ctx.C, ctx.region_of, ctx.comm), None, None, None, None, None, None, None

    @staticmethod
    def vmap(info: Any, in_dims: tuple, g: torch.Tensor, h: int, w: int, group: Any, R: int, C: int, region_of: Any, comm: Any) -> tuple:
        gb = to_front(g, in_dims[0])
        return _ScatterRegion.apply(gb, h, w, group, R, C, region_of, comm), (None if in_dims[0] is None else 0)


def fetch_region(x: torch.Tensor, group: dist.ProcessGroup, R: int, C: int, region_of: Any, comm: CommOp | str = "auto") -> torch.Tensor:
    """See :class:`_FetchRegion`; ``region_of(rank) -> (r0, r1, c0, c1)`` must be the same function on
    every rank (each rank also derives from it what the others read from its block)."""
    if group.size() == 1:
        r0, r1, c0, c1 = region_of(0)
        return x[..., r0:r1, c0:c1]
    return _FetchRegion.apply(x, group, R, C, region_of, comm)


def _local_product(a: torch.Tensor, b: torch.Tensor, a_t: bool, b_t: bool) -> torch.Tensor:
    """``op(a) @ op(b)``; on CUDA under bf16 the tcgen05 GEMM reads either operand in either major order, so
    no transposed copy is made."""
    if a.is_cuda and a.dim() == 2 and b.dim() == 2:
        from ...ops import linear_fused

        out = linear_fused.maybe_fused_matmul(a, b, a_t, b_t)
        if out is not None:
            return out
    return torch.matmul(a.transpose(-1, -2) if a_t else a, b.transpose(-1, -2) if b_t else b)


def block_matmul(kind: str, x: torch.Tensor, w: torch.Tensor, group: dist.ProcessGroup | None, R: int, C: int,
                 comm: CommOp | str = "auto") -> torch.Tensor:
    """Generic block product for a bare model group (the ``DistributedMatMul*`` modules).  ``group=None`` is a
    single process that holds both operands whole."""
    x, w = cast_to_autocast_dtype(x, w)
    if kind not in ("xwt", "xw", "xtw"):
        raise ValueError(kind)
    if group is None:
        return _local_product(x, w, kind == "xtw", kind == "xwt")
    xh, xw_, wh, ww = x.shape[-2], x.shape[-1], w.shape[-2], w.shape[-1]
    if kind == "xwt":          # X (M/R, K/C), W (N/R, K/C): rows i of X, the N/C rows of W that make output block j
        n = wh * R // C
        X = fetch_region(x, group, R, C, lambda p: ((p // C) * xh, (p // C + 1) * xh, 0, xw_ * C), comm)
        W = fetch_region(w, group, R, C, lambda p: ((p % C) * n, (p % C + 1) * n, 0, ww * C), comm)
        return _local_product(X, W, False, True)
    if kind == "xw":           # X (M/R, K/C), W (K/R, N/C): rows i of X, columns j of W
        X = fetch_region(x, group, R, C, lambda p: ((p // C) * xh, (p // C + 1) * xh, 0, xw_ * C), comm)
        W = fetch_region(w, group, R, C, lambda p: (0, wh * R, (p % C) * ww, (p % C + 1) * ww), comm)
        return _local_product(X, W, False, False)
    if kind == "xtw":          # X (K/R, M/C), W (K/R, N/C): the M/R columns of X that make output row block i, columns j of W
        m = xw_ * C // R
        X = fetch_region(x, group, R, C, lambda p: (0, xh * R, (p // C) * m, (p // C + 1) * m), comm)
        W = fetch_region(w, group, R, C, lambda p: (0, wh * R, (p % C) * ww, (p % C + 1) * ww), comm)
        return _local_product(X, W, True, False)
    raise ValueError(kind)
