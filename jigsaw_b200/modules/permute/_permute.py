"""``permute`` of a tensor whose two tracked axes are sharded over the ``row`` and ``col`` groups.

When the permutation swaps the two tracked axes, the data must be re-sharded: the axis that
was split over ``row`` ends up in the position sharded by ``col`` and vice versa.

* Swap path (any ``R x C`` grid whose ``mesh["model"]`` group is the row-major product of the two
  groups): the block a rank holds afterwards is a rectangle of the global matrix, so every rank
  fetches exactly that rectangle, piece by piece from the ranks that own it, in one sparse exchange
  over the chosen transport (``fetch_region``); each element travels once, nothing is gathered.
* General path (no usable ``model`` group): each tracked axis is gathered over the group that splits it
  and narrowed to the block the other group's rank owns.

Both are built from differentiable exchanges, so (unlike the reference, which is forward-only) the
permutation also back-propagates.

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
    comm = resolve_comm_op(comm, torch.device(device))
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
    model = mesh["model"] if "model" in mesh else None
    A, B = x.shape[row_dim] * R, x.shape[col_dim] * C           # global extents of the tracked axes
    if B % R:
        raise ValueError(f"axis {col_dim} (size {B}) doesn't divide evenly over {R} row ranks")
    if A % C:
        raise ValueError(f"axis {row_dim} (size {A}) doesn't divide evenly over {C} col ranks")
    if model is not None and model.size() == R * C and model.rank() == row.rank() * C + col.rank():
        # tracked axes to the back (a local permutation), fetch the rectangle this rank holds after the swap,
        # then the requested order: output position k takes the input axis dims[k], and the two tracked input
        # axes now sit at n - 2 (row_dim's) and n - 1 (col_dim's)
        rest = [d for d in range(n) if d not in (row_dim, col_dim)]
        z = x.permute(*rest, row_dim, col_dim)
        a, b = z.shape[-2], z.shape[-1]                         # local extents: A / R and B / C
        ha, hb = a * R // C, b * C // R                         # extents of the rectangle: A / C and B / R

        def region(p: int) -> tuple[int, int, int, int]:
            i, j = p // C, p % C
            return (j * ha, (j + 1) * ha, i * hb, (i + 1) * hb)

        from ..linear._functional import fetch_region

        z = fetch_region(z, model, R, C, region, comm)
        where = {d: k for k, d in enumerate(rest)}
        where[row_dim], where[col_dim] = n - 2, n - 1
        return z.permute(*(where[d] for d in dims)).contiguous()
    x = all_gather_cat(x.contiguous(), col, col_dim)
    x = all_gather_cat(x, row, row_dim)
    if x.shape[col_dim] % R:
        raise ValueError(f"axis {col_dim} (size {x.shape[col_dim]}) doesn't divide evenly over {R} row ranks")
    if x.shape[row_dim] % C:
        raise ValueError(f"axis {row_dim} (size {x.shape[row_dim]}) doesn't divide evenly over {C} col ranks")
    bc, br = x.shape[col_dim] // R, x.shape[row_dim] // C
    x = x.narrow(col_dim, row.rank() * bc, bc).narrow(row_dim, col.rank() * br, br)
    return x.permute(*dims).contiguous()
