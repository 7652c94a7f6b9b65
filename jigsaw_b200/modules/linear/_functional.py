"""2-D block-distributed matrix products as compositions of differentiable collectives.

Grid R x C, rank ``(i, j) = i * C + j`` of the model group.  Every operand and result is
block-distributed over its LAST TWO dimensions exactly as ``gather_results`` reassembles
them; leading dimensions are batch.

    XWT : Y = X  W^T   X (M/R, K/C)   W (N/R, K/C)   ->  Y (M/R, N/C)
    XW  : Y = X  W     X (M/R, K/C)   W (K/R, N/C)   ->  Y (M/R, N/C)
    XTW : Y = X^T W    X (K/R, M/C)   W (K/R, N/C)   ->  Y (M/R, N/C)

Schedule: all-gather -> GEMM.  The operand blocks a rank needs are gathered over the grid
axes, the local product is one GEMM; the backward (reduce-scatter of the operand
gradients) follows from the adjoints of the collectives.

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


class _GatherBlocks(torch.autograd.Function):
    """All-gather the ``R x C`` blocks of the last two dims over the model group; the
    backward sums the full-matrix gradients and keeps this rank's block."""

    @staticmethod
    def forward(ctx: Any, x: torch.Tensor, group: dist.ProcessGroup, R: int, C: int) -> torch.Tensor:
        ctx.group, ctx.R, ctx.C = group, R, C
        x = x.contiguous()
        parts = [torch.empty_like(x) for _ in range(R * C)]
        dist.all_gather(parts, x, group=group)
        rows = [torch.cat(parts[i * C : (i + 1) * C], dim=-1) for i in range(R)]
        return torch.cat(rows, dim=-2)

    @staticmethod
    def backward(ctx: Any, g: torch.Tensor) -> tuple:
        g = g.contiguous().clone()
        dist.all_reduce(g, op=dist.ReduceOp.SUM, group=ctx.group)
        r = ctx.group.rank()
        i, j = divmod(r, ctx.C)
        h, w = g.shape[-2] // ctx.R, g.shape[-1] // ctx.C
        return g[..., i * h : (i + 1) * h, j * w : (j + 1) * w].contiguous(), None, None, None


def gather_blocks(x: torch.Tensor, group: dist.ProcessGroup, R: int, C: int) -> torch.Tensor:
    if group.size() == 1:
        return x
    return _GatherBlocks.apply(x, group, R, C)


def _own_block(y: torch.Tensor, group: dist.ProcessGroup, R: int, C: int) -> torch.Tensor:
    i, j = divmod(group.rank(), C)
    h, w = y.shape[-2] // R, y.shape[-1] // C
    return y[..., i * h : (i + 1) * h, j * w : (j + 1) * w]


def block_matmul(kind: str, x: torch.Tensor, w: torch.Tensor, group: dist.ProcessGroup, R: int, C: int) -> torch.Tensor:
    """Generic block product for a bare model group (the ``DistributedMatMul*`` modules)."""
    x, w = cast_to_autocast_dtype(x, w)
    i, j = divmod(group.rank(), C)
    X = gather_blocks(x, group, R, C)
    W = gather_blocks(w, group, R, C)
    if kind == "xwt":
        m, n = X.shape[-2] // R, W.shape[-2] // C
        return torch.matmul(X[..., i * m : (i + 1) * m, :], W[..., j * n : (j + 1) * n, :].transpose(-1, -2))
    if kind == "xw":
        m, n = X.shape[-2] // R, W.shape[-1] // C
        return torch.matmul(X[..., i * m : (i + 1) * m, :], W[..., :, j * n : (j + 1) * n])
    if kind == "xtw":
        m, n = X.shape[-1] // R, W.shape[-1] // C
        return torch.matmul(X[..., :, i * m : (i + 1) * m].transpose(-1, -2), W[..., :, j * n : (j + 1) * n])
    raise ValueError(kind)
