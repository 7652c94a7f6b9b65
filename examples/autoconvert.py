"""Convert a plain PyTorch model with ``convert_to_jigsaw`` and check it against the original.

The converter swaps every layer it knows (Linear, Conv / ConvTranspose 1-3d, LayerNorm, GroupNorm,
Softmax, ``jigsaw_b200.modules.Attention / Roll / MatMul*``) for its distributed twin and gives each
rank its shard of the weights.  Elementwise modules stay; unknown modules stay with a warning
(``on_unrecognized="raise"`` makes that an error); modules that mix along a dimension (pooling, batch
norm ...) raise unless ``non_safe=True``.  The converted model takes sharded inputs: "row" cuts the
width / sequence, "col" the channels.

    torchrun --nproc-per-node 4 examples/autoconvert.py

Counterpart of the reference tutorial examples/autoconvert.py.
"""

import copy

import torch
from torch import nn

from _common import setup, shard

import jigsaw_b200 as jb
from jigsaw_b200.convert import convert_to_jigsaw
from jigsaw_b200.gather import gather_1d_results


class PatchMLP(nn.Module):
    """Patch embedding, a token MLP, patch recovery."""

    def __init__(self, channels=4, dim=64, patch=4):
        super().__init__()
        self.embed = nn.Conv2d(channels, dim, patch, stride=patch)
        self.fc1, self.act, self.fc2 = nn.Linear(dim, 4 * dim), nn.GELU(), nn.Linear(4 * dim, dim)
        self.recover = nn.ConvTranspose2d(dim, channels, patch, stride=patch)

    def forward(self, x):
        z = self.embed(x)
        b, e, h, w = z.shape
        z = z.permute(0, 2, 3, 1).reshape(b, h * w, e)
        z = z + self.fc2(self.act(self.fc1(z)))
        return self.recover(z.reshape(b, h, w, e).permute(0, 3, 1, 2))


class TinyTransformer(nn.Module):
    """The same with a pre-norm attention block in the middle."""

    def __init__(self, device, channels=4, dim=64, heads=4, patch=4):
        super().__init__()
        self.embed = nn.Conv2d(channels, dim, patch, stride=patch, device=device)
        self.norm1, self.norm2 = nn.LayerNorm(dim, device=device), nn.LayerNorm(dim, device=device)
        self.attn = jb.modules.Attention(dim, dim, dim, heads, device)
        self.fc1, self.act, self.fc2 = nn.Linear(dim, 4 * dim, device=device), nn.GELU(), nn.Linear(4 * dim, dim, device=device)
        self.recover = nn.ConvTranspose2d(dim, channels, patch, stride=patch, device=device)

    def forward(self, x):
        z = self.embed(x)
        b, e, h, w = z.shape
        z = z.permute(0, 2, 3, 1).reshape(b, h * w, e).contiguous()
        z = z + self.attn(self.norm1(z))
        z = z + self.fc2(self.act(self.fc1(self.norm2(z))))
        return self.recover(z.reshape(b, h, w, e).permute(0, 3, 1, 2).contiguous())


def check(name, reference, model, mesh, device, rel):
    row, col = mesh["row"], mesh["col"]
    x = torch.randn(2, 4, 32, 64, device=device)
    x_local = shard(shard(x, 1, col), -1, row)
    with torch.no_grad():
        expected = reference(x)
        out = gather_1d_results(gather_1d_results(model(x_local), mesh, dim=1, pm_key="col"), mesh, dim=-1, pm_key="row")
    err = (out - expected).abs().max().item()
    jb.log.info("%s: forward max |converted - original| = %.2e (max |original| = %.2e)", name, err, expected.abs().max())
    assert err <= rel * expected.abs().max().item() + 1e-5, err
    reference(x).square().mean().backward()
    jb.modules.DistributedMSELoss(reduce_groups=(row, col))(model(x_local), torch.zeros_like(x_local)).backward()
    ref = reference.fc1.weight.grad                   # (4E, E): rows over "row", columns over "col"
    nr, nc = ref.shape[0] // row.size(), ref.shape[1] // col.size()
    ref = ref[row.rank() * nr:(row.rank() + 1) * nr, col.rank() * nc:(col.rank() + 1) * nc]
    gerr = ((model.fc1.weight.grad - ref).abs().max() / ref.abs().max()).item()
    jb.log.info("%s: backward max relative error of the fc1.weight.grad shard = %.2e", name, gerr)
    assert gerr < max(rel, 1e-4), gerr


def main() -> None:
    device, rank, world = setup()
    jb.launch.setup_precision(tf32=False)             # compare in true fp32
    mesh = jb.make_process_mesh({"row": 2, "col": 2})
    torch.manual_seed(0)                              # same seed: every rank builds the same full model
    reference = PatchMLP().to(device)
    model = convert_to_jigsaw(copy.deepcopy(reference), mesh, device)
    jb.log.info("converted layers: %s", [type(m).__name__ for m in model.children()])
    check("PatchMLP", reference, model, mesh, device, 1e-4)
    plain = model.fc1.convert_to_torch(mesh)          # and back: a plain nn.Linear on every rank
    torch.testing.assert_close(plain.weight, reference.fc1.weight)
    torch.testing.assert_close(plain.bias, reference.fc1.bias)

    torch.manual_seed(1)
    reference2 = TinyTransformer(device)
    model2 = convert_to_jigsaw(copy.deepcopy(reference2), mesh, device)
    jb.log.info("converted layers: %s", [type(m).__name__ for m in model2.children()])
    # on CUDA the attention core computes in half precision even for fp32 inputs
    check("TinyTransformer", reference2, model2, mesh, device, 5e-3 if device.type == "cuda" else 1e-4)


if __name__ == "__main__":
    main()
