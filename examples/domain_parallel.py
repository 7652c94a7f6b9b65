"""Domain parallelism only: a small encoder-decoder CNN on an image cut into 2x2 tiles.

Every rank holds all weights and one tile ``(B, C, H / sh, W / sw)``.  A 3x3 convolution needs one
row / column of its neighbours' pixels: ``DistributedConv2d`` fetches that halo, the strided
convolution halves the map, ``DistributedConvTranspose2d`` doubles it again (its outputs overlap the
tile border, so it *adds* a halo into the neighbours), ``DistributedGroupNorm`` reduces its statistics
over the tiles, and ``DistributedMSELoss`` averages over all pixels of all tiles.  Gradients of the
replicated weights are summed over the tiles inside the backward pass.

    torchrun --nproc-per-node 4 examples/domain_parallel.py
    torchrun --nproc-per-node 8 examples/domain_parallel.py --ddp        # two copies, plain DDP over "dp"
    torchrun --nproc-per-node 8 examples/domain_parallel.py --joint-hook # one all-reduce per bucket

Counterpart of the reference tutorial examples/domain_parallel.py.
"""

import sys

from torch import nn

from _common import ddp_flags, denoising_batch, setup, shard, steps_flag, train

import jigsaw_b200 as jb

H, W, CH = 64, 64, 2


def build_model(mesh, device) -> nn.Module:
    kw = dict(device=device, spatial_group=(mesh["sh"], mesh["sw"]), channel_group=mesh["col"])
    M = jb.modules

    def norm(c):
        return M.DistributedGroupNorm(4, c, device, channel_group=mesh["col"], spatial_group=(mesh["sh"], mesh["sw"]))

    return nn.Sequential(
        M.DistributedConv2d(CH, 16, 3, padding=1, **kw), norm(16), nn.GELU(),
        M.DistributedConv2d(16, 32, 3, stride=2, padding=1, **kw), norm(32), nn.GELU(),
        M.DistributedConvTranspose2d(32, 16, 4, stride=2, padding=1, **kw), norm(16), nn.GELU(),
        M.DistributedConv2d(16, CH, 3, padding=1, **kw),
    )


def main(steps: int = 100, data_parallel: bool = False, joint_hook: bool = False) -> list[float]:
    device, rank, world = setup()
    axes = {"sh": 2, "sw": 2, "col": 1}
    mesh = (jb.make_process_mesh({"dp": -1, **axes}, model_parallel_axes=tuple(axes)) if data_parallel
            else jb.make_process_mesh(axes))
    jb.launch.set_all_seeds(0)                       # replicated weights: the same seed everywhere
    model = build_model(mesh, device)
    if data_parallel:
        model = jb.parallel.wrap_ddp(model, mesh, joint_hook=joint_hook)
    loss_fn = jb.modules.DistributedMSELoss(reduce_groups=(mesh["sh"], mesh["sw"]))

    def batch(step):
        return tuple(shard(shard(t, -2, mesh["sh"]), -1, mesh["sw"]).to(device)
                     for t in denoising_batch(step, mesh, (4, CH, H, W)))

    return train(model, loss_fn, batch, steps)


if __name__ == "__main__":
    main(**ddp_flags(sys.argv), **steps_flag(sys.argv))
