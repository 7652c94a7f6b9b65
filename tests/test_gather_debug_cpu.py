"""Helpers around a sharded model: averaging replicas, gathering tiles, counting parameters.

Reference behaviours covered: tests/test_gather.py (replica averaging, ``bias_only``), tests/test_debug.py
(parameter counts with frozen parameters, with a mesh, with a data-parallel axis, with and without bias).
"""

import pytest
import torch

from dist_utils import all_ok, assert_close, run_distributed, split


def test_count_parameters_leaves_out_frozen_ones():
    from jigsaw_b200 import debug

    model = torch.nn.Sequential(torch.nn.Linear(3, 2), torch.nn.LayerNorm(2))
    assert debug.count_parameters(model) == 6 + 2 + 2 + 2
    model[0].bias.requires_grad_(False)
    model[1].weight.requires_grad_(False)
    assert debug.count_parameters(model) == 6 + 2


def _worker_averaging(rank, world):
    import torch.distributed as dist
    from jigsaw_b200 import gather

    group = dist.group.WORLD
    # replicas that agree are left as they are, None entries are passed over
    same = [torch.full((2,), 3.0), torch.arange(4.0)]
    gather.average_weights([same[0], None, same[1]], group)
    assert_close(same[0], torch.full((2,), 3.0), "identical replicas", 0, 0)
    assert_close(same[1], torch.arange(4.0), "identical replicas", 0, 0)
    # replicas that differ meet in the middle
    mine = torch.full((3,), float(rank))
    gather.average_weights([mine], group)
    assert_close(mine, torch.full((3,), (world - 1) / 2), "mean over ranks", 0, 0)
    # bias_only touches nothing else
    layer = torch.nn.Linear(2, 2)
    with torch.no_grad():
        layer.weight.fill_(float(rank))
        layer.bias.fill_(float(rank))
    gather.average_weights_module(layer, group, bias_only=True)
    assert_close(layer.bias.data, torch.full((2,), (world - 1) / 2), "bias averaged", 0, 0)
    assert bool((layer.weight == float(rank)).all())
    gather.average_weights_module(layer, group)
    assert_close(layer.weight.data, torch.full((2, 2), (world - 1) / 2), "weight averaged", 0, 0)
    # the same over a sub-group: only its members mix
    import jigsaw_b200 as jb

    mesh = jb.make_process_mesh({"row": 2, "col": 2})
    t = torch.full((1,), float(rank))
    gather.average_weights([t], mesh["col"])
    members = dist.get_process_group_ranks(mesh["col"])
    assert_close(t, torch.full((1,), sum(members) / len(members)), "mean over the column group", 0, 0)


def test_replica_averaging():
    run_distributed(_worker_averaging, 4, timeout=300)


def _worker_gathers(rank, world):
    import jigsaw_b200 as jb
    from jigsaw_b200 import gather

    mesh = jb.make_process_mesh({"row": 2, "col": 2})
    torch.manual_seed(3)
    full = torch.randn(2, 6, 8)
    tile = split(full, {1: mesh["row"], 2: mesh["col"]})
    assert_close(gather.gather_results(tile, mesh), full, "2-D gather", 0, 0)
    tiles = gather.gather_results_as_list(tile, mesh)
    assert len(tiles) == 4
    for r in range(2):
        for c in range(2):
            assert_close(tiles[r * 2 + c], full[:, 3 * r:3 * r + 3, 4 * c:4 * c + 4], f"tile ({r}, {c}) of the list", 0, 0)
    assert len(gather.gather_results_as_list(tile)) == world                              # no mesh: the world group
    strip = split(full, {1: mesh["row"]})
    assert_close(gather.gather_1d_results(strip, mesh, dim=1, pm_key="row"), full, "1-D gather", 0, 0)
    pieces = gather.gather_1d_results_list(strip, mesh, pm_key="row")
    assert [tuple(p.shape) for p in pieces] == [(2, 3, 8)] * 2
    assert_close(torch.cat(pieces, 1), full, "1-D list", 0, 0)
    # other axis names
    alias = {"tok": mesh["row"], "chan": mesh["col"], "mp": mesh["model"]}
    assert_close(gather.gather_results(tile, alias, "tok", "chan", "mp"), full, "2-D gather, other names", 0, 0)


def test_gathers_of_tiles_and_strips():
    run_distributed(_worker_gathers, 4, timeout=300)


def _worker_counts(rank, world, data_parallel, bias):
    """Tiles are summed, a bias that the row ranks hold alike is counted once, and so are data-parallel copies."""
    import jigsaw_b200 as jb
    from jigsaw_b200 import debug

    mesh = (jb.make_process_mesh({"dp": 2, "row": 2, "col": 1}, model_parallel_axes=("row", "col")) if data_parallel
            else jb.make_process_mesh({"row": 2, "col": 2}))
    layer = jb.modules.DistributedLinear(6, 8, "cpu", mesh["model"], mesh["row"], mesh["col"], bias=bias)
    total = debug.count_parameters(layer, mesh)
    assert all_ok(total == 6 * 8 + (8 if bias else 0)), total
    assert debug.count_parameters(layer) == layer.weight.numel() + (layer.bias.numel() if bias else 0)
    layer.weight.requires_grad_(False)
    assert all_ok(debug.count_parameters(layer, mesh) == (8 if bias else 0))


@pytest.mark.parametrize("data_parallel", [False, True])
@pytest.mark.parametrize("bias", [True, False])
def test_count_parameters_with_a_mesh_is_the_whole_model(data_parallel, bias):
    run_distributed(_worker_counts, 4, data_parallel, bias, timeout=300)
