"""Training on copies x tiles gives the model that one process gives on the whole batch.

Eight ranks train the Swin model as two data-parallel copies of 2 x 2 tiles, each copy on half of the global
batch; the oracle is the same model on a mesh of one rank, trained on the whole batch (every rank computes it).
Loss curve and weight updates must agree.  This pins the scale of the loss: the tile sum of the replicated
gradients and the mean over the copies only give the gradient of the global mean when each rank back-propagates
the copy's mean loss as seen from its tile: a loss that reduces over the tiles, or the local mean divided by the
number of tiles.  The undivided local mean is too large by that number and must be caught.  The optimizer is SGD
with momentum, because Adam divides the scale out.

Reference behaviours covered: tests/test_ddp_serial.py (both accepted losses), tests/test_ddp_mutation.py:88-98
(the unscaled loss and the missing sum are noticed).
"""

import pytest
import torch
import torch.nn.functional as F

from dist_utils import all_ok, run_distributed, singleton_mesh, split

STEPS, BATCH, LR, REL = 6, 4, 0.05, 1e-4


def _batch(step, cfg):
    gen = torch.Generator().manual_seed(100 + step)
    shape = (BATCH, cfg.in_channels, *cfg.image_size)
    return torch.randn(shape, generator=gen), torch.randn(shape, generator=gen)


def _train_cut(loss_kind, cfg):
    import torch.distributed as dist

    import jigsaw_b200 as jb
    from jigsaw_b200 import checkpoint
    from jigsaw_b200.models import Swin

    mesh = jb.make_process_mesh({"dp": 2, "sh": 2, "sw": 2, "col": 1}, model_parallel_axes=("sh", "sw", "col"))
    tiles = (mesh["sh"], mesh["sw"])
    n_tiles = tiles[0].size() * tiles[1].size()
    jb.launch.set_all_seeds(0)
    model = Swin(mesh, "cpu", cfg)
    start = checkpoint.full_state_dict(model)
    ddp = jb.parallel.wrap_ddp(model, mesh)
    opt = torch.optim.SGD(ddp.parameters(), lr=LR, momentum=0.9)
    mse = jb.modules.DistributedMSELoss(reduce_groups=tiles)
    per_copy = BATCH // mesh["dp"].size()
    mine = slice(mesh["dp"].rank() * per_copy, (mesh["dp"].rank() + 1) * per_copy)
    cuts = {2: mesh["sh"], 3: mesh["sw"]}
    curve = []
    for step in range(STEPS):
        x, y = (split(t[mine], cuts) for t in _batch(step, cfg))
        out = ddp(x)
        if loss_kind == "over_tiles":
            loss = mse(out, y)
        else:
            loss = F.mse_loss(out, y) / (n_tiles if loss_kind == "local_scaled" else 1)
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
        seen = loss.detach().clone()
        if loss_kind == "local_unscaled":
            seen /= n_tiles
        if loss_kind != "over_tiles":                                  # the copy's loss is the sum over its tiles
            dist.all_reduce(seen, group=mesh["model"])
        dist.all_reduce(seen, group=mesh["dp"])
        curve.append(float(seen) / mesh["dp"].size())
    return curve, start, checkpoint.full_state_dict(model)


def _train_whole(start, cfg):
    from jigsaw_b200 import checkpoint
    from jigsaw_b200.models import Swin

    model = Swin(singleton_mesh("sh", "sw", "col"), "cpu", cfg)
    checkpoint.load_full_state_dict(model, start)
    opt = torch.optim.SGD(model.parameters(), lr=LR, momentum=0.9)
    curve = []
    for step in range(STEPS):
        x, y = _batch(step, cfg)
        loss = F.mse_loss(model(x), y)
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
        curve.append(float(loss))
    return curve, {k: v.detach() for k, v in model.state_dict().items()}


def _worker(rank, world, loss_kind, sync_on, expect_match):
    import jigsaw_b200.parallel._sync as sync
    from jigsaw_b200.models import SwinConfig

    cfg = SwinConfig(image_size=(32, 32), in_channels=1, patch=2, dims=(8, 16), heads=(2, 4), depths=(2, 2), window=4)
    sync._SYNC_DISABLED = not sync_on
    curve, start, final = _train_cut(loss_kind, cfg)
    sync._SYNC_DISABLED = False
    want_curve, want_final = _train_whole(start, cfg)
    got, want = torch.tensor(curve), torch.tensor(want_curve)
    problems = []
    if not torch.allclose(got, want, rtol=REL, atol=REL * float(want.abs().max())):
        problems.append(f"loss curve {curve} against {want_curve}")
    for name, first in start.items():
        if not first.is_floating_point():
            continue
        update, want_update = final[name] - first, want_final[name] - first             # updates are small beside the weights
        if not torch.allclose(update, want_update, rtol=REL, atol=REL * float(want_update.abs().max()) + 1e-7):
            problems.append(f"update of {name}: off by {float((update - want_update).abs().max()):.3e}")
    matched = all_ok(not problems)
    assert matched == expect_match, (loss_kind, sync_on, problems[:3])


@pytest.mark.parametrize("loss_kind", ["over_tiles", "local_scaled"])
def test_copies_of_tiles_train_like_one_process(loss_kind):
    run_distributed(_worker, 8, loss_kind, True, True, timeout=900)


def test_undivided_local_loss_is_caught():
    run_distributed(_worker, 8, "local_unscaled", True, False, timeout=900)


def test_missing_tile_sum_is_caught():
    run_distributed(_worker, 8, "over_tiles", False, False, timeout=900)
