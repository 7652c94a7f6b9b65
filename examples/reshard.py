"""Move a trained model onto another mesh, or gather it into plain PyTorch.

Train a two-layer MLP whose weights are cut over both axes of a 2x2 mesh, then
(1) ``convert_to_torch`` every layer: a plain ``nn.Sequential`` that needs no jigsaw_b200,
(2) ``reshard_parameters`` onto a mesh of 4 full replicas (one per rank, e.g. for serving),
(3) ``checkpoint.save_sharded`` on the training mesh and ``load_sharded`` on a 1x4 mesh.

    torchrun --nproc-per-node 4 examples/reshard.py

Counterpart of the reference tutorial examples/reshard.py ((3) has no counterpart there).
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


def main(steps: int = 100) -> None:
    device, rank, world = setup()
    train_mesh = jb.make_process_mesh({"row": 2, "col": 2})
    row, col = train_mesh["row"], train_mesh["col"]
    jb.launch.set_all_seeds(train_mesh["model"].rank())
    model = mlp(train_mesh, device)
    opt = torch.optim.Adam(model.parameters(), lr=1e-2)
    loss_fn = jb.modules.DistributedMSELoss(reduce_groups=(row, col))

    def local(x, mesh=train_mesh):
        return shard(shard(x, 1, mesh["row"]), 2, mesh["col"]).to(device)

    for step in range(steps):
        x = torch.randn(4, 8, DIM, generator=torch.Generator().manual_seed(step))
        loss = loss_fn(model(local(x)), local(torch.tanh(x)))
        opt.zero_grad()
        loss.backward()
        opt.step()
    jb.log.info("trained: loss %.4f", loss.item())
    x_test = torch.randn(2, 8, DIM, generator=torch.Generator().manual_seed(1234))
    with torch.no_grad():
        expected = jb.gather.gather_results(model(local(x_test)), train_mesh)

    plain = nn.Sequential(model[0].convert_to_torch(train_mesh), nn.GELU(), model[2].convert_to_torch(train_mesh))
    with torch.no_grad():
        err = (plain(x_test.to(device)) - expected).abs().max().item()
    jb.log.info("plain nn.Sequential vs distributed: max diff %.2e", err)
    assert err < 1e-4, err

    holder = [tempfile.mkdtemp() if rank == 0 else None]
    dist.broadcast_object_list(holder, src=0)
    jb.checkpoint.save_sharded(model, train_mesh, holder[0])
    wide = jb.make_process_mesh({"row": 1, "col": 4})
    other = mlp(wide, device)
    jb.checkpoint.load_sharded(other, wide, holder[0])
    with torch.no_grad():
        out = jb.gather.gather_results(other(local(x_test, wide)), wide)
    err = (out - expected).abs().max().item()
    jb.log.info("checkpoint read back on a 1x4 mesh: max diff %.2e", err)
    assert err < 1e-4, err

    infer_mesh = jb.make_process_mesh({"dp": 4, "row": 1, "col": 1}, model_parallel_axes=("row", "col"))
    for layer in model.modules():
        if hasattr(layer, "reshard_parameters"):
            layer.reshard_parameters(train_mesh, infer_mesh)
    with torch.no_grad():
        err = (model(x_test.to(device)) - expected).abs().max().item()    # nothing is cut: full inputs
    jb.log.info("resharded onto 4 replicas: max diff %.2e", err)
    assert err < 1e-4, err


if __name__ == "__main__":
    main(**steps_flag(sys.argv))
