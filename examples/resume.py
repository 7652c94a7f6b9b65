"""Stop a run, change the mesh, carry on: a checkpoint with optimizer state read back on another mesh.

An MLP whose weights are cut over both axes of a 2x2 mesh trains for some steps (each step accumulates
two micro-batches with a single gradient reduction), writes ``checkpoint.save_sharded(..., optimizer=opt)``,
and a fresh model and optimizer on a 1x4 mesh continue from it.  The continued run must land where an
uninterrupted run on the first mesh lands.

    torchrun --nproc-per-node 4 examples/resume.py

No counterpart in the reference (its recipe stops at one state dict per model rank).
"""

import sys
import tempfile

import torch
import torch.distributed as dist
from torch import nn

from _common import setup, shard, steps_flag

import jigsaw_b200 as jb

DIM = 32


def mlp(mesh, device):
    def linear(i, o):
        return jb.modules.DistributedLinear(i, o, device, mesh["model"], mesh["row"], mesh["col"])

    return nn.Sequential(linear(DIM, 4 * DIM), nn.GELU(), linear(4 * DIM, DIM))


def train(model, opt, mesh, device, first: int, last: int) -> float:
    loss_fn = jb.modules.DistributedMSELoss(reduce_groups=(mesh["row"], mesh["col"]))

    def local(x):
        return shard(shard(x, 1, mesh["row"]), 2, mesh["col"]).to(device)

    total = 0.0
    for step in range(first, last):
        opt.zero_grad()
        with jb.parallel.no_grad_sync():                         # two micro-batches, gradients stay local ...
            for micro in range(2):
                x = torch.randn(4, 8, DIM, generator=torch.Generator().manual_seed(2 * step + micro))
                loss = loss_fn(model(local(x)), local(torch.tanh(x))) / 2
                loss.backward()
                total = loss.item() * 2
        jb.parallel.reduce_replica_grads(model)                  # ... and are summed over their copies once
        opt.step()
    return total


def main(steps: int = 40) -> None:
    device, rank, world = setup()
    half = steps // 2
    first_mesh = jb.make_process_mesh({"row": 2, "col": 2})
    jb.launch.set_all_seeds(first_mesh["model"].rank())
    model = mlp(first_mesh, device)
    start = jb.checkpoint.full_state_dict(model)
    opt = jb.optim.FusedAdam(model.parameters(), lr=1e-2)

    loss = train(model, opt, first_mesh, device, 0, half)
    holder = [tempfile.mkdtemp() if rank == 0 else None]
    dist.broadcast_object_list(holder, src=0)
    jb.checkpoint.save_sharded(model, first_mesh, holder[0], extra={"next_step": half}, optimizer=opt)
    jb.log.info("step %d: loss %.4f, checkpoint in %s", half, loss, holder[0])

    wide = jb.make_process_mesh({"row": 1, "col": 4})
    resumed = mlp(wide, device)
    opt2 = jb.optim.FusedAdam(resumed.parameters(), lr=1.0)      # the saved hyper-parameters replace these
    extra = jb.checkpoint.load_sharded(resumed, wide, holder[0], optimizer=opt2)
    loss = train(resumed, opt2, wide, device, extra["next_step"], steps)
    jb.log.info("step %d on the 1x4 mesh: loss %.4f", steps, loss)

    straight = mlp(first_mesh, device)
    jb.checkpoint.load_full_state_dict(straight, start)
    train(straight, jb.optim.FusedAdam(straight.parameters(), lr=1e-2), first_mesh, device, 0, steps)
    want, got = jb.checkpoint.full_state_dict(straight), jb.checkpoint.full_state_dict(resumed)
    err = max((want[k] - got[k]).abs().max().item() for k in want)
    jb.log.info("resumed vs uninterrupted: max parameter difference %.2e", err)
    assert err < 1e-4, err


if __name__ == "__main__":
    main(**steps_flag(sys.argv))
