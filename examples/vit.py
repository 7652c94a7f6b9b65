"""Vision Transformer with domain *and* tensor parallelism (``jigsaw_b200.models.ViT``).

The 2x2 mesh cuts every tensor twice: image ``(B, C / col, H, W / row)``, tokens
``(B, N / row, E / col)``.  Attention is global: ring attention passes key/value chunks around "row"
(``--ulysses`` swaps it for the all-to-all scheme: heads are scattered, sequences gathered), heads are
split over "col", the MLP weights over both axes, layer-norm statistics are reduced over "col".

    torchrun --nproc-per-node 4 examples/vit.py [--ulysses]
    torchrun --nproc-per-node 8 examples/vit.py --ddp | --joint-hook

Parameters come in two kinds.  MLP weights are cut over "row" and "col" (a different block on every
rank of a copy): only averaged over "dp".  Everything else is cut over "col" at most and equal along
"row", where each rank saw other tokens: summed over "row" (by the layers, in the backward pass), then
averaged over "dp".  ``wrap_ddp`` builds a DDP over "dp" only and checks the set-up.

Counterpart of the reference tutorial examples/vit.py.
"""

import sys

from _common import ddp_flags, denoising_batch, setup, shard, steps_flag, train

import jigsaw_b200 as jb
from jigsaw_b200.models import ViT, ViTConfig

CFG = ViTConfig(image_size=(32, 64), in_channels=4, patch=4, dim=64, heads=4, depth=2)


def local_batch(step, mesh, device, batch=4):
    H, W = CFG.image_size
    return tuple(shard(shard(t, 1, mesh["col"]), -1, mesh["row"]).to(device)
                 for t in denoising_batch(step, mesh, (batch, CFG.in_channels, H, W)))


def build(device, data_parallel=False, joint_hook=False, ulysses=False):
    if data_parallel:
        mesh = jb.make_process_mesh({"dp": -1, "row": 2, "col": 2}, model_parallel_axes=("row", "col"))
    else:
        mesh = jb.make_process_mesh({"row": 2, "col": 2})
    jb.launch.set_all_seeds(mesh["model"].rank())     # sharded weights: a different seed per model rank
    cfg = ViTConfig(**{**CFG.__dict__, "sequence_parallel": "ulysses" if ulysses else "ring"})
    model = ViT(mesh, device, cfg)
    if data_parallel:
        model = jb.parallel.wrap_ddp(model, mesh, joint_hook=joint_hook)
    return mesh, model


def main(steps: int = 100, data_parallel: bool = False, joint_hook: bool = False, ulysses: bool = False) -> list[float]:
    device, rank, world = setup()
    mesh, model = build(device, data_parallel, joint_hook, ulysses)
    jb.log.info("parameters: %d on this rank, %d in the model", jb.debug.count_parameters(model),
                jb.debug.count_parameters(model, mesh))
    loss_fn = jb.modules.DistributedMSELoss(reduce_groups=(mesh["row"], mesh["col"]))
    return train(model, loss_fn, lambda s: local_batch(s, mesh, device), steps)


if __name__ == "__main__":
    main(ulysses="--ulysses" in sys.argv, **ddp_flags(sys.argv), **steps_flag(sys.argv))
