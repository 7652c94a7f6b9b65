"""Swin Transformer with domain parallelism (``jigsaw_b200.models.Swin``): window attention needs no ring.

Tiles hold whole windows, so attention, patch merging, MLP and norms are local; only the half-window
shift of every second block (``DistributedRoll``) talks to the neighbouring tiles.  The shifted-window
mask is built from the tile's global position.  Weights are replicated over the tiles; their gradients
are summed over the tiles in the backward pass.

    torchrun --nproc-per-node 4 examples/swin.py
    torchrun --nproc-per-node 8 examples/swin.py --ddp | --joint-hook

Counterpart of the reference tutorial examples/swin.py.
"""

import sys

from _common import ddp_flags, denoising_batch, setup, shard, steps_flag, train

import jigsaw_b200 as jb
from jigsaw_b200.models import Swin, SwinConfig

CFG = SwinConfig(image_size=(64, 64), in_channels=1, patch=2, dims=(32, 64), heads=(2, 4), depths=(2, 2), window=4)


def main(steps: int = 100, data_parallel: bool = False, joint_hook: bool = False) -> list[float]:
    device, rank, world = setup()
    axes = {"sh": 2, "sw": 2, "col": 1}
    mesh = (jb.make_process_mesh({"dp": -1, **axes}, model_parallel_axes=tuple(axes)) if data_parallel
            else jb.make_process_mesh(axes))
    jb.launch.set_all_seeds(0)
    model = Swin(mesh, device, CFG)
    if data_parallel:
        model = jb.parallel.wrap_ddp(model, mesh, joint_hook=joint_hook)
    loss_fn = jb.modules.DistributedMSELoss(reduce_groups=(mesh["sh"], mesh["sw"]))

    def batch(step):
        return tuple(shard(shard(t, -2, mesh["sh"]), -1, mesh["sw"]).to(device)
                     for t in denoising_batch(step, mesh, (4, CFG.in_channels, *CFG.image_size)))

    return train(model, loss_fn, batch, steps)


if __name__ == "__main__":
    main(**ddp_flags(sys.argv), **steps_flag(sys.argv))
