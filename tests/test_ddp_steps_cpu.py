"""Replicas hold the same bits after every one of many optimizer steps.

A tile sum that is slightly off gives replicas slightly different gradients; one step may hide that, AdamW's
normalisation blows it up over the next ones.  So each layer kind is trained for a dozen steps through
``wrap_ddp`` and after every ``optimizer.step()`` each parameter is compared bit for bit over its replica groups
and over the data-parallel axis.  With the tile sum switched off the replicas must part on a mesh that has
tiles, and nothing may change on a mesh that has none.

Reference behaviours covered: tests/test_ddp_steps.py (identity after every step, parameters moved and finite),
tests/test_ddp_mutation.py:74-86 (the check fails without the sum; a mesh without replicas is unaffected).
"""

import pytest
import torch

from dist_utils import all_ok, run_distributed
from test_ddp_variants_cpu import KINDS, _build, _identical_over

STEPS = 12
MESHES = {"2x2x2": (2, 2, 2), "2x2x1": (2, 2, 1), "2x1x2": (2, 1, 2), "4x1x1": (4, 1, 1)}


def _train(shape, kind, steps):
    """Returns the first step at which some parameter differed between replicas (None if never), and whether
    every parameter moved and stayed finite."""
    import jigsaw_b200 as jb

    mesh = jb.make_process_mesh(dict(zip(("dp", "row", "col"), shape)), model_parallel_axes=("row", "col"))
    layer, make_input = _build(kind, mesh)
    with torch.no_grad():
        for p in layer.parameters():
            p.mul_(0.1)                                          # the integer start would saturate the softmax
    ddp = jb.parallel.wrap_ddp(layer, mesh)
    opt = torch.optim.AdamW(ddp.parameters(), lr=1e-2)
    first = [p.detach().clone() for p in layer.parameters()]
    parted = None
    for step in range(steps):
        opt.zero_grad(set_to_none=True)
        ddp(make_input(step)).float().pow(2).mean().backward()
        opt.step()
        same = True
        for p in layer.parameters():
            for grp in jb.parallel.replica_groups(p):
                same &= _identical_over(p.detach(), grp)
            same &= _identical_over(p.detach(), mesh["dp"])
        if not all_ok(same):                                     # agreed over all ranks, so every rank stops at the same step
            parted = step
            break
        jb.debug.assert_replica_consistency(layer, mesh)
    healthy = all(bool(torch.isfinite(p).all()) and not torch.equal(p.detach(), b) for p, b in zip(layer.parameters(), first))
    return parted, healthy


def _worker_identity(rank, world, shape):
    for kind in KINDS:
        parted, healthy = _train(shape, kind, STEPS)
        assert parted is None, f"{shape} {kind}: replicas differ after step {parted}"
        assert all_ok(healthy), f"{shape} {kind}: a parameter never moved or is not finite"


@pytest.mark.parametrize("shape", list(MESHES.values()), ids=list(MESHES))
def test_replicas_stay_identical(shape):
    run_distributed(_worker_identity, shape[0] * shape[1] * shape[2], shape, timeout=900)


def _worker_without_sum(rank, world, shape, must_part):
    import jigsaw_b200.parallel._sync as sync

    sync._SYNC_DISABLED = True
    for kind in KINDS:
        parted, _ = _train(shape, kind, 2)
        if must_part:
            assert parted == 0, f"{shape} {kind}: replicas still agree after a step without the tile sum"
        else:
            assert parted is None, f"{shape} {kind}: a mesh without replicas must not depend on the switch"


def test_replicas_part_at_once_without_the_tile_sum():
    run_distributed(_worker_without_sum, 4, (2, 2, 1), True, timeout=600)


def test_a_mesh_without_tiles_does_not_need_the_sum():
    run_distributed(_worker_without_sum, 4, (4, 1, 1), False, timeout=600)
