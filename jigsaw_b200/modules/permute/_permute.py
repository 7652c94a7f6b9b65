"""``permute`` of a tensor whose two tracked axes are sharded over the ``row`` and ``col`` groups.

When the permutation swaps the two tracked axes, the data must be re-sharded: the axis that
was split over ``row`` ends up in the position sharded by ``col`` and vice versa.  Each
tracked axis is gathered over the group that splits it and narrowed to the block the other
group's rank owns.  Built from differentiable collectives, so (unlike the reference, which
is forward-only) it also back-propagates.

Reference parity: jigsaw/modules/permute/_distributed_permute.py:58-295 (swap kernels for
1x2 / 2x2 / 4x2), :300-407 (dispatch and general path).
"""

from __future__ import annotations

from collections.abc import Mapping, Sequence

import torch
import torch.distributed as dist

from ..._core.collectives import all_gather_cat
from ..._core.comm import CommOp, resolve_comm_op


def distributed_permute(
    x: torch.Tensor,
    dims: Sequence[int],
    row_dim: int,
    col_dim: int,
    local_rank: int | None,
    device: torch.device | str,
    mesh: Mapping[str, dist.ProcessGroup],
    comm: CommOp | str = CommOp.AUTO,
) -> torch.Tensor:
    """Permute ``x`` by ``dims``; ``mesh["row"]`` shards position ``row_dim`` and ``mesh["col"]``
    position ``col_dim`` in both input and output.  ``dims`` must map those two positions onto
    themselves, unchanged or swapped."""
    resolve_comm_op(comm, torch.device(device))
    dims = tuple(dims)
    n = x.dim()
    if sorted(dims) != list(range(n)):
        raise ValueError(f"dims {dims} is not a permutation of range({n})")
    if row_dim == col_dim or not 0 <= row_dim < n or not 0 <= col_dim < n:
        raise ValueError(f"row_dim {row_dim} and col_dim {col_dim} must be distinct axes of a {n}-d tensor")
    if {dims[row_dim], dims[col_dim]} != {row_dim, col_dim}:
        raise ValueError(
            f"dims {dims} moves an axis other than row_dim={row_dim}/col_dim={col_dim} into one of those "
            "two positions (or moves one of them out); distributed_permute only knows how to reshard those "
            "two axes; the others may be sharded by a mesh it has no knowledge of"
        )
    if dims[row_dim] == row_dim:
        return x.permute(*dims).contiguous()
    row, col = mesh["row"], mesh["col"]
    R, C = row.size(), col.size()
    x = all_gather_cat(x.contiguous(), col, col_dim)
    x = all_gather_cat(x, row, row_dim)
    if x.shape[col_dim] % R:
        raise ValueError(f"axis {col_dim} (size {x.shape[col_dim]}) doesn't divide evenly over {R} row ranks")
    if x.shape[row_dim] % C:
        raise ValueError(f"axis {row_dim} (size {x.shape[row_dim]}) doesn't divide evenly over {C} col ranks")
    bc, br = x.shape[col_dim] // R, x.shape[row_dim] // C
    x = x.narrow(col_dim, row.rank() * bc, bc).narrow(row_dim, col.rank() * br, br)
    return x.permute(*dims).contiguous()
