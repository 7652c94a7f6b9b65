"""``convert_to_jigsaw`` on whole models: what comes out computes what went in.

A transformer block written with plain torch modules and this library's single-device ``Attention`` is converted
onto a 2 x 2 mesh (tokens over the rows, features over the columns) and compared with the original: output, input
gradient, and every parameter gradient gathered back to the original's shape.  Smaller cases cover the layer kinds
one by one: softmax over the cut feature axis, layer norm without affine parameters, group norm, the products of
two activations, roll, and a (transposed) convolution pair.

Reference behaviours covered: tests/test_convert.py (linear, MLP, attention, transformer block, convolutions, roll,
matmul, group norm, softmax, layer norm without affine parameters).
"""

import copy

import pytest
import torch

from dist_utils import all_ok, assert_close, run_distributed, split


class _Block(torch.nn.Module):
    """Pre-norm transformer block on ``(batch, tokens, features)``."""

    def __init__(self, dim, heads):
        super().__init__()
        from jigsaw_b200.modules.attention import Attention

        self.norm1 = torch.nn.LayerNorm(dim)
        self.attn = Attention(dim, dim, dim, heads, "cpu", attn_backend="math")
        self.norm2 = torch.nn.LayerNorm(dim)
        self.mlp = torch.nn.Sequential(torch.nn.Linear(dim, 4 * dim), torch.nn.GELU(), torch.nn.Linear(4 * dim, dim))

    def forward(self, x):
        x = x + self.attn(self.norm1(x))
        return x + self.mlp(self.norm2(x))


def _worker_block(rank, world, sequence_parallel):
    import jigsaw_b200 as jb
    from jigsaw_b200 import checkpoint, convert

    mesh = jb.make_process_mesh({"row": 2, "col": 2})
    torch.manual_seed(0)
    serial = _Block(16, 4).double()
    x = torch.randn(2, 8, 16, dtype=torch.float64)
    cuts = {1: mesh["row"], 2: mesh["col"]}
    kwargs = {"ring": sequence_parallel == "ring", "ulysses": sequence_parallel == "ulysses", "attn_backend": "math"}
    sharded = convert.convert_to_jigsaw(copy.deepcopy(serial), mesh, "cpu", **kwargs)
    M = jb.modules
    assert isinstance(sharded.attn, M.DistributedAttention) and isinstance(sharded.norm1, M.DistributedLayerNorm)
    assert isinstance(sharded.mlp[0], M.DistributedLinear) and isinstance(sharded.mlp[1], torch.nn.GELU)
    assert (sharded.attn.ring, sharded.attn.ulysses) == (kwargs["ring"], kwargs["ulysses"])
    xr = x.clone().requires_grad_(True)
    want = serial(xr)
    seed = torch.randn(want.shape, generator=torch.Generator().manual_seed(1), dtype=torch.float64)
    want.backward(seed)
    xl = split(x, cuts).requires_grad_(True)
    got = sharded(xl)
    assert_close(got, split(want.detach(), cuts), f"{sequence_parallel}: output", 1e-9, 1e-9)
    got.backward(split(seed, cuts))
    assert_close(xl.grad, split(xr.grad, cuts), f"{sequence_parallel}: input gradient", 1e-9, 1e-9)
    # gradients in the original's layout: put them in the parameters' place and gather like a state dict
    back = copy.deepcopy(serial)
    for p in sharded.parameters():
        p.data, p.grad = p.grad, None
    checkpoint.load_full_state_dict(back, checkpoint.full_state_dict(sharded))
    for (name, g), (_, p) in zip(back.named_parameters(), serial.named_parameters()):
        assert_close(g.data, p.grad, f"{sequence_parallel}: gradient of {name}", 1e-8, 1e-9)


@pytest.mark.parametrize("sequence_parallel", ["ring", "ulysses"])
def test_transformer_block(sequence_parallel):
    run_distributed(_worker_block, 4, sequence_parallel, timeout=300)


def _worker_kinds(rank, world):
    import jigsaw_b200 as jb
    from jigsaw_b200 import convert

    mesh = jb.make_process_mesh({"row": 2, "col": 2})
    M, row, col = jb.modules, mesh["row"], mesh["col"]
    gen = torch.Generator().manual_seed(3)
    tokens = torch.randn(2, 8, 16, generator=gen, dtype=torch.float64)
    cuts = {1: row, 2: col}
    # softmax over the feature axis, which the columns cut
    for dim in (-1, 2):
        soft = convert.convert_to_jigsaw(torch.nn.Sequential(torch.nn.Softmax(dim=dim)), mesh, "cpu")[0]
        assert isinstance(soft, M.DistributedSoftmax)
        assert_close(soft(split(tokens, cuts)), split(torch.softmax(tokens, -1), cuts), f"softmax dim={dim}", 1e-12, 1e-12)
        assert isinstance(soft.convert_to_torch(), torch.nn.Softmax) and soft.convert_to_torch().dim == dim
    with pytest.raises(NotImplementedError, match="explicit dim"):
        convert.convert_to_jigsaw(torch.nn.Sequential(torch.nn.Softmax()), mesh, "cpu")
    # layer norm without affine parameters: nothing to shard, statistics still span the columns
    ln = convert.convert_to_jigsaw(torch.nn.Sequential(torch.nn.LayerNorm(16, elementwise_affine=False)), mesh, "cpu")[0]
    assert isinstance(ln, M.DistributedLayerNorm) and not list(ln.parameters())
    want = torch.nn.functional.layer_norm(tokens, (16,))
    assert_close(ln(split(tokens, cuts)), split(want, cuts), "layer norm without affine parameters", 1e-9, 1e-9)
    assert not list(ln.convert_to_torch(mesh).parameters())
    # group norm: channels over the columns, width over the rows
    torch.manual_seed(4)
    gn_ref = torch.nn.GroupNorm(4, 8).double()
    with torch.no_grad():
        gn_ref.weight.uniform_(0.5, 1.5)
        gn_ref.bias.uniform_(-0.5, 0.5)
    image = torch.randn(2, 8, 6, 8, generator=gen, dtype=torch.float64)
    image_cuts = {1: col, 3: row}
    gn = convert.convert_to_jigsaw(torch.nn.Sequential(copy.deepcopy(gn_ref)), mesh, "cpu")[0]
    assert isinstance(gn, M.DistributedGroupNorm)
    assert_close(gn(split(image, image_cuts)), split(gn_ref(image).detach(), image_cuts), "group norm", 1e-9, 1e-9)
    back = gn.convert_to_torch(mesh)
    assert_close(back.weight.data, gn_ref.weight.data, "group norm weight back", 0, 0)
    # a convolution followed by its transposed counterpart
    torch.manual_seed(5)
    pair_ref = torch.nn.Sequential(torch.nn.Conv2d(8, 8, 3, stride=2, padding=1), torch.nn.GELU(),
                                   torch.nn.ConvTranspose2d(8, 8, 4, stride=2, padding=1)).double()
    pair = convert.convert_to_jigsaw(copy.deepcopy(pair_ref), mesh, "cpu")
    assert isinstance(pair[0], M.DistributedConv2d) and isinstance(pair[2], M.DistributedConvTranspose2d)
    assert_close(pair(split(image, image_cuts)), split(pair_ref(image).detach(), image_cuts), "conv then transposed conv", 1e-9, 1e-9)
    # the products of two activations: a model that owns none of the operands
    class Scores(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.qk, self.av = M.MatMulXWT(), M.MatMulXW()

        def forward(self, q, k, v):
            return self.av(torch.softmax(self.qk(q, k), -1), v)

    scores = convert.convert_to_jigsaw(Scores(), mesh, "cpu")
    assert isinstance(scores.qk, M.DistributedMatMulXWT) and isinstance(scores.av, M.DistributedMatMulXW)
    assert scores.qk.model_group is mesh["model"]
    # roll along the token axis that the rows cut
    # (the converter takes axis -2 to be the one the rows cut unless ``dim_to_mesh_axis`` says otherwise)
    for dims, extra in (((-2,), {}), ((1,), {"dim_to_mesh_axis": {1: "row"}})):
        roll = convert.convert_to_jigsaw(torch.nn.Sequential(M.Roll((3,), dims, dtype=torch.float64)), mesh, "cpu", **extra)[0]
        assert isinstance(roll, M.DistributedRoll)
        assert_close(roll(split(tokens, cuts)), split(torch.roll(tokens, 3, 1), cuts), f"roll over the cut token axis, dims={dims}", 0, 0)
    assert all_ok(True)


def test_layer_kinds_one_by_one():
    run_distributed(_worker_kinds, 4, timeout=300)


def _worker_cast_after_construction(rank, world):
    """A module cast with ``.double()`` / ``.to(dtype)`` after it was built converts in the dtype of its weights, in
    both directions."""
    import jigsaw_b200 as jb
    from jigsaw_b200.modules.attention import Attention

    mesh = jb.make_process_mesh({"row": 2, "col": 2})
    torch.manual_seed(0)                                                                      # the same module on every rank
    serial = Attention(8, 8, 8, 2, "cpu", attn_backend="math", qk_norm=True).double()        # built in float32, then cast
    sharded = Attention.convert_to_jigsaw(serial, mesh, "cpu", attn_backend="math")
    assert all(p.dtype == torch.float64 for p in sharded.parameters())
    back = sharded.convert_to_torch(mesh)
    assert all(p.dtype == torch.float64 for p in back.parameters())
    assert_close(back.qkv.weight.data, serial.qkv.weight.data, "qkv weight there and back", 0, 0)
    halved = Attention.convert_to_jigsaw(Attention(8, 8, 8, 2, "cpu").to(torch.bfloat16), mesh, "cpu")
    assert all(p.dtype == torch.bfloat16 for p in halved.parameters())
    assert all(p.dtype == torch.bfloat16 for p in halved.to(torch.float32).to(torch.bfloat16).convert_to_torch(mesh).parameters())


def test_modules_cast_after_construction_convert_in_their_weights_dtype():
    run_distributed(_worker_cast_after_construction, 4, timeout=300)
