"""The rest of a data-parallel training loop, on the ViT of ``vit.py`` (2x2 model mesh, "dp" copies on top).

* The **global batch** is cut over "dp"; the ranks of one copy read the same images and keep their shard.
* **Gradient accumulation**: each copy's share runs in micro-batches; ``no_sync()`` holds DDP's
  all-reduce back until the last one and every micro-batch loss is divided by their number.
* The **joint hook** (default; ``--plain`` turns it off) reduces each replicated gradient over
  ``dp x row`` in DDP's buckets: same gradients, one collective fewer.
* The **logged loss** is the mean over the copies.
* A **replica check** (``assert_replica_consistency``) every few steps raises on every rank if a
  replicated weight has drifted apart, the symptom of a gradient that is not summed over its copies.
* **Checkpoint**: ``jigsaw_b200.checkpoint.save_sharded`` writes one file per model shard (copies do not
  write), the optimizer's moments cut the same way, and a manifest that any other mesh can load.

    torchrun --nproc-per-node 8 examples/ddp.py        # 4 ranks also run: a single copy

Counterpart of the reference tutorial examples/ddp.py.
"""

import contextlib
import sys
import tempfile

import torch
import torch.distributed as dist

from _common import setup, shard, steps_flag
from vit import CFG, build

import jigsaw_b200 as jb

GLOBAL_BATCH, MICRO_BATCH, CHECK_EVERY = 8, 2, 25


def my_share(t: torch.Tensor, mesh, device) -> torch.Tensor:
    t = shard(t, 0, mesh["dp"])                                           # images over the copies
    return shard(shard(t, 1, mesh["col"]), -1, mesh["row"]).to(device)    # then channels and width


def train_step(ddp, opt, loss_fn, x, y, mesh) -> float:
    chunks = list(zip(x.split(MICRO_BATCH), y.split(MICRO_BATCH)))
    opt.zero_grad(set_to_none=True)
    total = torch.zeros((), device=x.device)
    for i, (xm, ym) in enumerate(chunks):
        hold = contextlib.nullcontext() if i == len(chunks) - 1 else ddp.no_sync()
        with hold:
            loss = loss_fn(ddp(xm), ym) / len(chunks)
            loss.backward()
        total += loss.detach()
    opt.step()
    dist.all_reduce(total, group=mesh["dp"])
    return total.item() / mesh["dp"].size()


def main(steps: int = 100, joint_hook: bool = True) -> list[float]:
    device, rank, world = setup()
    mesh, ddp = build(device, data_parallel=True, joint_hook=joint_hook)
    if GLOBAL_BATCH % (mesh["dp"].size() * MICRO_BATCH):
        raise ValueError(f"{mesh['dp'].size()} copies cannot cut {GLOBAL_BATCH} images into micro-batches of {MICRO_BATCH}")
    opt = torch.optim.AdamW(ddp.parameters(), lr=1e-3)
    loss_fn = jb.modules.DistributedMSELoss(reduce_groups=(mesh["row"], mesh["col"]))
    losses = []
    for step in range(steps):
        g = torch.Generator().manual_seed(step)                     # the global batch: same on every rank
        clean = torch.nn.functional.avg_pool2d(torch.randn(GLOBAL_BATCH, CFG.in_channels, *CFG.image_size, generator=g), 5, 1, 2)
        noisy = clean + 0.3 * torch.randn(clean.shape, generator=g)
        losses.append(train_step(ddp, opt, loss_fn, my_share(noisy, mesh, device), my_share(clean, mesh, device), mesh))
        if step % CHECK_EVERY == 0 or step == steps - 1:
            jb.debug.assert_replica_consistency(ddp, mesh)          # collective over the whole mesh
        if step % 20 == 0:
            jb.log.info("step %3d  loss %.4f", step, losses[-1])
    holder = [tempfile.mkdtemp() if rank == 0 else None]
    dist.broadcast_object_list(holder, src=0)
    jb.checkpoint.save_sharded(ddp.module, mesh, holder[0], extra={"steps": steps}, optimizer=opt)
    jb.log.info("checkpoint with one file per model shard in %s", holder[0])
    return losses


if __name__ == "__main__":
    main(joint_hook="--plain" not in sys.argv, **steps_flag(sys.argv))
