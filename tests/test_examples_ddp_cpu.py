"""The data-parallel tutorial's training step is exact, and its log is the same on every rank.

``examples/ddp.py`` gives each copy of the model half of the global batch, runs it in two micro-batches under
``no_sync()`` with each loss divided by their number, and lets DDP average over the copies.  The oracle is a second
model with the same weights on the same 2 x 2 model mesh that takes the whole batch in one pass, without DDP.
Loss curve and weight updates must agree, with the joint hook and without (SGD with momentum, so that a wrong
scale is not divided out).

Reference behaviours covered: tests/test_examples_ddp.py:106-122 (every rank logs the global loss), :278-320
(the tutorial's step against the full batch).
"""

import os
import sys

import pytest
import torch

from dist_utils import all_ok, run_distributed

EXAMPLES = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples")
STEPS, LR, REL = 4, 0.05, 1e-4


def _tutorial():
    import importlib

    import torch.distributed as dist

    if EXAMPLES not in sys.path:
        sys.path.insert(0, EXAMPLES)
    common = importlib.import_module("_common")
    common.setup = lambda: (torch.device("cpu"), dist.get_rank(), dist.get_world_size())
    module = importlib.import_module("ddp")
    module.setup = common.setup
    return module


def _worker_step(rank, world, joint_hook):
    import jigsaw_b200 as jb
    from jigsaw_b200.models import ViT

    ddp_example = _tutorial()
    cfg = ddp_example.CFG
    mesh = jb.make_process_mesh({"dp": 2, "row": 2, "col": 2}, model_parallel_axes=("row", "col"))
    assert ddp_example.GLOBAL_BATCH // mesh["dp"].size() // ddp_example.MICRO_BATCH == 2, "the test wants two micro-batches"
    models = []
    for _ in range(2):
        jb.launch.set_all_seeds(mesh["model"].rank())
        models.append(ViT(mesh, "cpu", cfg))
    model, whole = models
    first = [p.detach().clone() for p in model.parameters()]
    wrapped = jb.parallel.wrap_ddp(model, mesh, joint_hook=joint_hook)
    opt = torch.optim.SGD(wrapped.parameters(), lr=LR, momentum=0.9)
    whole_opt = torch.optim.SGD(whole.parameters(), lr=LR, momentum=0.9)
    loss_fn = jb.modules.DistributedMSELoss(reduce_groups=(mesh["row"], mesh["col"]))
    one_copy = {"dp": _Single(), "row": mesh["row"], "col": mesh["col"]}
    curve, whole_curve = [], []
    for step in range(STEPS):
        gen = torch.Generator().manual_seed(step)
        x = torch.randn(ddp_example.GLOBAL_BATCH, cfg.in_channels, *cfg.image_size, generator=gen)
        y = torch.randn(x.shape, generator=gen)
        curve.append(ddp_example.train_step(wrapped, opt, loss_fn, ddp_example.my_share(x, mesh, "cpu"),
                                            ddp_example.my_share(y, mesh, "cpu"), mesh))
        loss = loss_fn(whole(ddp_example.my_share(x, one_copy, "cpu")), ddp_example.my_share(y, one_copy, "cpu"))
        whole_opt.zero_grad(set_to_none=True)
        loss.backward()
        whole_opt.step()
        whole_curve.append(float(loss))
    got, want = torch.tensor(curve), torch.tensor(whole_curve)
    problems = []
    if not torch.allclose(got, want, rtol=REL, atol=REL * float(want.abs().max())):
        problems.append(f"loss curve {curve} against {whole_curve}")
    for (name, p), q, p0 in zip(model.named_parameters(), whole.parameters(), first):
        update, want_update = p.detach() - p0, q.detach() - p0
        if not torch.allclose(update, want_update, rtol=REL, atol=REL * float(want_update.abs().max()) + 1e-7):
            problems.append(f"update of {name} off by {float((update - want_update).abs().max()):.3e}")
    assert all_ok(not problems), problems[:3]
    jb.debug.assert_replica_consistency(model, mesh)


class _Single:
    """Stands for a data-parallel axis with one copy: the whole batch stays."""

    def size(self):
        return 1

    def rank(self):
        return 0


@pytest.mark.parametrize("joint_hook", [False, True], ids=["plain", "joint"])
def test_tutorial_step_matches_the_whole_batch(joint_hook):
    run_distributed(_worker_step, 8, joint_hook, timeout=900)


def _worker_log(rank, world):
    import torch.distributed as dist

    losses = torch.tensor(_tutorial().main(steps=3), dtype=torch.float64)
    assert bool(torch.isfinite(losses).all())
    on_rank_0 = losses.clone()
    dist.broadcast(on_rank_0, src=0)
    assert all_ok(torch.equal(losses, on_rank_0)), "ranks log different losses"


def test_every_rank_logs_the_global_loss():
    run_distributed(_worker_log, 8, timeout=900)
