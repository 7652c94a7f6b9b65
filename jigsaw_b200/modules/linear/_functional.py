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

Region = tuple[int, int, int, int]          # rows [r0, r1) and columns [c0, c1) of the global matrix


def _overlap(a: Region, b: Region) -> Region | None:
    r0, r1, c0, c1 = max(a[0], b[0]), min(a[1], b[1]), max(a[2], b[2]), min(a[3], b[3])
    return (r0, r1, c0, c1) if r0 < r1 and c0 < c1 else None


def _transport(comm: CommOp | str, device: torch.device) -> CommOp:
    try:
        return resolve_comm_op(comm, device)
    except ValueError:                      # a transport chosen for another device type
        return resolve_comm_op("auto", device)


class _FetchRegion(torch.autograd.Function):
    """``region_of(rank)`` of a matrix whose last two dimensions are cut into ``R x C`` blocks over
    ``group`` (rank ``i * C + j`` holds block ``(i, j)``): every rank receives its region piece by piece
    from the owners of the blocks it overlaps.  Backward: the adjoint scatter-add."""

    @staticmethod
    def forward(ctx: Any, x: torch.Tensor, group: dist.ProcessGroup, R: int, C: int, region_of: Any, comm: Any) -> torch.Tensor:
        x = x.contiguous()
        h, w = x.shape[-2], x.shape[-1]
        me = group.rank()
        block = lambda p: ((p // C) * h, (p // C + 1) * h, (p % C) * w, (p % C + 1) * w)  # noqa: E731
        mine, want = block(me), region_of(me)
        lead = x.shape[:-2]
        out = x.new_empty(*lead, want[1] - want[0], want[3] - want[2])
        sends, recvs, places = {}, {}, {}
        plan_send, plan_recv = {}, {}
        for p in range(R * C):
            give = _overlap(region_of(p), mine)                # part of my block that rank p reads
            if give is not None:
                plan_send[p] = give
                sends[p] = x[..., give[0] - mine[0]:give[1] - mine[0], give[2] - mine[2]:give[3] - mine[2]].contiguous()
            take = _overlap(want, block(p))                    # part of rank p's block that I read
            if take is not None:
                plan_recv[p] = take
                recvs[p] = x.new_empty(*lead, take[1] - take[0], take[3] - take[2])
                places[p] = (slice(take[0] - want[0], take[1] - want[0]), slice(take[2] - want[2], take[3] - want[2]))
        comm = _transport(comm, x.device)
        sparse_exchange(sends, recvs, group, comm)
        for p, buf in recvs.items():
            out[(..., *places[p])] = buf
        ctx.group, ctx.comm, ctx.mine, ctx.want = group, comm, mine, want
        ctx.plan_send, ctx.plan_recv, ctx.places, ctx.x_shape, ctx.x_dtype = plan_send, plan_recv, places, x.shape, x.dtype
        return out

    @staticmethod
    def backward(ctx: Any, g: torch.Tensor) -> tuple:
        mine = ctx.mine
        lead = ctx.x_shape[:-2]
        sends = {p: g[(..., *ctx.places[p])].contiguous() for p in ctx.plan_recv}
        recvs = {p: g.new_empty(*lead, give[1] - give[0], give[3] - give[2]) for p, give in ctx.plan_send.items()}
        sparse_exchange(sends, recvs, ctx.group, ctx.comm)
        acc = torch.zeros(ctx.x_shape, dtype=torch.promote_types(g.dtype, torch.float32), device=g.device)
        for p, give in ctx.plan_send.items():
            acc[..., give[0] - mine[0]:give[1] - mine[0], give[2] - mine[2]:give[3] - mine[2]] += recvs[p]
        return acc.to(ctx.x_dtype), None, None, None, None, None


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


def block_matmul(kind: str, x: torch.Tensor, w: torch.Tensor, group: dist.ProcessGroup, R: int, C: int,
                 comm: CommOp | str = "auto") -> torch.Tensor:
    """Generic block product for a bare model group (the ``DistributedMatMul*`` modules)."""
    x, w = cast_to_autocast_dtype(x, w)
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
