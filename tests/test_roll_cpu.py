"""``Roll`` / ``DistributedRoll`` beyond the parity check of the layer sweep: transports, validation, re-sharding of
the layout, conversion back to the serial layer, gradients (the adjoint roll), ``vmap``, shifts larger than a tile.

Reference behaviours covered: tests/modules/roll/test_roll_module.py:28-56 (transport selection), :58-99 (serial
layer, gradients, parameter count, conversion, configs, vmap), :100-124 (validation, re-sharding),
tests/modules/roll/test_roll.py (2x2 and 4x2 tilings).
"""

import pytest
import torch

from dist_utils import assert_close, run_distributed, split


def test_serial_roll_and_validation():
    from jigsaw_b200.modules import DistributedRoll, Roll, RollConfig

    x = torch.arange(24.0).view(2, 3, 4)
    roll = Roll((1, -2), (1, 2))
    assert torch.equal(roll(x), torch.roll(x, (1, -2), (1, 2))) and roll.get_parameter_count() == 0
    xr = x.clone().requires_grad_(True)
    g = torch.randn(2, 3, 4)
    roll(xr).backward(g)
    assert torch.equal(xr.grad, torch.roll(g, (-1, 2), (1, 2)))            # the gradient is rolled back
    assert str(RollConfig(device="cpu").comm) in ("auto", "batch_isend_irecv")
    with pytest.raises(ValueError):
        RollConfig(device="cpu", comm="carrier_pigeon")
    with pytest.raises(ValueError):
        RollConfig(device="cpu", comm="all_to_all")                       # needs CUDA
    with pytest.raises(ValueError, match="must align"):
        DistributedRoll((1,), (0,), (0,), (), "cpu")
    with pytest.raises(ValueError, match="must appear in dims"):
        DistributedRoll((1,), (0,), (1,), (None,), "cpu")
    layer = DistributedRoll((1, 2), (0, 2), (0,), (None,), "cpu")
    with pytest.raises(ValueError, match="mismatched lengths"):
        layer.reshard([0], [])
    layer.reshard([0, 2], [None, None])
    assert tuple(layer.distributed_dims) == (0, 2) and len(layer.spatial_groups) == 2
    assert torch.equal(layer(x), torch.roll(x, (1, 2), (0, 2)))           # nothing is split: a plain roll
    back = layer.convert_to_torch()
    assert isinstance(back, Roll) and torch.equal(back(x), torch.roll(x, (1, 2), (0, 2)))


def _worker_roll(rank, world, R, C):
    import jigsaw_b200 as jb
    from jigsaw_b200.modules import DistributedRoll, RollConfig

    mesh = jb.make_process_mesh({"row": R, "col": C})
    row, col = mesh["row"], mesh["col"]
    g = torch.Generator().manual_seed(0)
    x = torch.randn(2, 8 * R, 8 * C, 3, generator=g, dtype=torch.float64)
    cuts = {1: row, 2: col}
    for comm in ("auto", "isend", "batch_isend_irecv"):
        for shifts in ((3, -2), (-8, 8), (0, 5), (11, -13)):              # inside a tile, exactly one tile, mixed, beyond a tile
            layer = DistributedRoll(shifts, (1, 2), (1, 2), (row, col), "cpu", dtype=torch.float64, config=RollConfig(device="cpu", comm=comm))
            xl = split(x, cuts).requires_grad_(True)
            y = layer(xl)
            assert_close(y, split(torch.roll(x, shifts, (1, 2)), cuts), f"{R}x{C} {comm} {shifts}: forward", 0, 0)
            gy = torch.randn(x.shape, generator=torch.Generator().manual_seed(1), dtype=torch.float64)
            y.backward(split(gy, cuts))
            assert_close(xl.grad, split(torch.roll(gy, (-shifts[0], -shifts[1]), (1, 2)), cuts), f"{R}x{C} {comm} {shifts}: gradient", 0, 0)
    # one rolled dimension is split, the other is not; vmap over a leading batch equals a loop
    layer = DistributedRoll((2, 1), (1, 3), (1,), (row,), "cpu", dtype=torch.float64)
    xl = split(x, {1: row})
    assert_close(layer(xl), split(torch.roll(x, (2, 1), (1, 3)), {1: row}), f"{R}x{C}: one split dimension", 0, 0)
    stack = torch.stack([xl, 2 * xl, -xl])
    shifted = DistributedRoll((2, 1), (1, 3), (1,), (row,), "cpu", dtype=torch.float64)
    got = torch.vmap(shifted)(stack)
    want = torch.stack([shifted(stack[i]) for i in range(3)])
    assert_close(got, want, f"{R}x{C}: vmap", 0, 0)
    assert "distributed_dims=(1,)" in repr(layer) and layer.get_parameter_count() == 0


@pytest.mark.parametrize("grid", [(2, 2), (4, 2)])
def test_roll_over_tiled_dimensions(grid):
    R, C = grid
    run_distributed(_worker_roll, R * C, R, C, timeout=300)
