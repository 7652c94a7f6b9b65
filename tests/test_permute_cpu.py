"""``distributed_permute``: swapping the two sharded axes on any grid over every CPU transport (forward and
gradient against ``torch.permute`` of the global tensor), tracked axes in any position, the gather path
for meshes without a model group.

Reference behaviours covered: tests/modules/permute/test_distributed_permute.py (swap kernels on 1x2, 2x2,
4x2 against the general path and against torch; argument checks are in tests/test_modules_cpu.py).
"""

import pytest
import torch

from dist_utils import assert_close, run_distributed, split


def _worker_permute(rank, world, R, C):
    import jigsaw_b200 as jb
    mesh = jb.make_process_mesh({"row": R, "col": C})
    row, col = mesh["row"], mesh["col"]
    f = jb.modules.functional.distributed_permute
    torch.manual_seed(0)
    L = R * C * 2
    for comm in ("auto", "isend", "batch_isend_irecv"):
        # trailing axes
        t = torch.randn(3, L, 2 * L, dtype=torch.float64)
        tl = split(t, {1: row, 2: col}).requires_grad_(True)
        out = f(tl, (0, 2, 1), 1, 2, None, "cpu", mesh, comm)
        assert_close(out, split(t.permute(0, 2, 1), {1: row, 2: col}), f"swap {R}x{C} {comm}", 0, 0)
        g = torch.randn(3, 2 * L, L, dtype=torch.float64)
        out.backward(split(g, {1: row, 2: col}))
        assert_close(tl.grad, split(g.permute(0, 2, 1), {1: row, 2: col}), f"swap grad {R}x{C} {comm}", 0, 0)
        # tracked axes in front and apart, other axes reordered too
        t = torch.randn(L, 3, 2 * L, 5, dtype=torch.float64)
        tl = split(t, {0: row, 2: col})
        out = f(tl, (2, 3, 0, 1), 0, 2, None, "cpu", mesh, comm)
        assert_close(out, split(t.permute(2, 3, 0, 1), {0: row, 2: col}), f"swap4d {R}x{C} {comm}", 0, 0)
        # col before row
        t = torch.randn(2 * L, L, dtype=torch.float64)
        tl = split(t, {1: row, 0: col})
        out = f(tl, (1, 0), 1, 0, None, "cpu", mesh, comm)
        assert_close(out, split(t.permute(1, 0), {1: row, 0: col}), f"swap colfirst {R}x{C} {comm}", 0, 0)
    # general path (no model group) agrees
    t = torch.randn(3, L, 2 * L, dtype=torch.float64)
    out = f(split(t, {1: row, 2: col}), (0, 2, 1), 1, 2, None, "cpu", {"row": row, "col": col})
    assert_close(out, split(t.permute(0, 2, 1), {1: row, 2: col}), f"general {R}x{C}", 0, 0)


@pytest.mark.parametrize("grid", [(1, 2), (2, 2), (2, 1), (3, 2), (4, 2)])
def test_swap_of_sharded_axes(grid):
    R, C = grid
    run_distributed(_worker_permute, R * C, R, C, timeout=300)
