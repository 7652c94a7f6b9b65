"""A standing diagnostic of the gradient synchronisation: at a fixed global batch the gradient does not depend on
how the work is cut.  Four ranks hold either four copies of the model with one image each, two copies with two
tiles per image, or one copy with four tiles; the gradients of the replicated weights must be the same in all
three, and with the tile sum switched off their norm must fall with the number of tiles.

Reference behaviours covered: tests/test_ddp_mutation.py:101-155 (gradient norm against the tiling, with and
without the synchronisation).
"""

import os
import sys

import torch

from dist_utils import all_ok, run_distributed, split

EXAMPLES = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples")
CUTS = ((4, 1, 1), (2, 2, 1), (1, 2, 2))                     # (copies, tiles along H, tiles along W)


def _gradients(cut, state):
    import jigsaw_b200 as jb

    if EXAMPLES not in sys.path:
        sys.path.insert(0, EXAMPLES)
    from domain_parallel import CH, H, W, build_model

    copies, sh, sw = cut
    mesh = jb.make_process_mesh({"dp": copies, "sh": sh, "sw": sw, "col": 1}, model_parallel_axes=("sh", "sw", "col"))
    model = build_model(mesh, torch.device("cpu"))
    if state is not None:
        model.load_state_dict(state)                         # every weight is held whole, so one state fits every cut
    else:
        state = {k: v.clone() for k, v in model.state_dict().items()}
    ddp = jb.parallel.wrap_ddp(model, mesh)
    gen = torch.Generator().manual_seed(0)
    x, y = torch.randn(4, CH, H, W, generator=gen), torch.randn(4, CH, H, W, generator=gen)
    per_copy = 4 // copies
    mine = slice(mesh["dp"].rank() * per_copy, (mesh["dp"].rank() + 1) * per_copy)
    tiles = {2: mesh["sh"], 3: mesh["sw"]}
    loss = jb.modules.DistributedMSELoss(reduce_groups=(mesh["sh"], mesh["sw"]))
    loss(ddp(split(x[mine], tiles)), split(y[mine], tiles)).backward()
    return torch.cat([p.grad.reshape(-1) for p in model.parameters()]), state


def _worker(rank, world, synchronised):
    import jigsaw_b200.parallel._sync as sync

    torch.manual_seed(0)
    sync._SYNC_DISABLED = not synchronised
    state, grads = None, []
    for cut in CUTS:
        g, state = _gradients(cut, state)
        grads.append(g)
    norms = [float(g.norm()) for g in grads]
    if synchronised:
        worst = max(float((g - grads[0]).abs().max()) for g in grads[1:])
        assert all_ok(worst <= 1e-5 * float(grads[0].abs().max())), (worst, norms)
        assert all_ok(all(abs(n - norms[0]) <= 1e-5 * norms[0] for n in norms)), norms
    else:
        assert all_ok(all(n < 0.9 * norms[0] for n in norms[1:])), norms


def test_gradient_does_not_depend_on_the_tiling():
    run_distributed(_worker, 4, True, timeout=600)


def test_gradient_norm_falls_with_the_tiles_when_the_sum_is_switched_off():
    run_distributed(_worker, 4, False, timeout=600)
