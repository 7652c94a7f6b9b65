"""3-D encoder-decoder on a volume cut over its two trailing axes (``jigsaw_b200.models.UNet3d``).

Strided ``DistributedConv3d`` layers fetch a halo plane, ``DistributedConvTranspose3d`` layers add one
into the neighbours, ``DistributedGroupNorm`` reduces its statistics over the tiles, and the loss is a
per-voxel binary cross-entropy over all tiles.

    torchrun --nproc-per-node 4 examples/unet3d.py
    torchrun --nproc-per-node 8 examples/unet3d.py --ddp | --joint-hook

The reference has the 3-D layers but no 3-D tutorial.
"""

import sys

import torch

from _common import data_seed, ddp_flags, setup, shard, steps_flag, train

import jigsaw_b200 as jb
from jigsaw_b200.models import UNet3d, UNet3dConfig

CFG = UNet3dConfig(widths=(8, 16), norm_groups=4)
D = H = W = 16


def main(steps: int = 100, data_parallel: bool = False, joint_hook: bool = False) -> list[float]:
    device, rank, world = setup()
    axes = {"sh": 2, "sw": 2, "col": 1}
    mesh = (jb.make_process_mesh({"dp": -1, **axes}, model_parallel_axes=tuple(axes)) if data_parallel
            else jb.make_process_mesh(axes))
    jb.launch.set_all_seeds(0)
    model = UNet3d(mesh, device, CFG)
    if data_parallel:
        model = jb.parallel.wrap_ddp(model, mesh, joint_hook=joint_hook)
    loss_fn = jb.modules.DistributedBCEWithLogitsLoss(reduce_groups=(mesh["sh"], mesh["sw"]))

    def batch(step):
        g = torch.Generator().manual_seed(data_seed(step, mesh))
        field = torch.nn.functional.avg_pool3d(torch.randn(2, 1, D, H, W, generator=g), 3, 1, 1)
        x, y = field + 0.2 * torch.randn(field.shape, generator=g), (field > 0).float()   # segment the smooth field
        return tuple(shard(shard(t, -2, mesh["sh"]), -1, mesh["sw"]).to(device) for t in (x, y))

    return train(model, loss_fn, batch, steps, lr=3e-3)


if __name__ == "__main__":
    main(**ddp_flags(sys.argv), **steps_flag(sys.argv))
