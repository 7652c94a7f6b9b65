"""``torch.vmap`` over the distributed layers (ensembles of inputs): the batched call must equal a
loop over the ensemble members, forward and gradients."""

import torch

from dist_utils import assert_close, run_distributed


def _worker_vmap(rank, world):
    import jigsaw_b200 as jb

    mesh = jb.make_process_mesh({"row": 2, "col": 2})
    row, col = mesh["row"], mesh["col"]
    torch.manual_seed(rank)
    lin = jb.modules.DistributedLinear(8, 12, "cpu", mesh["model"], row, col)
    norm = jb.modules.DistributedLayerNorm(12, None, "cpu", row, col)
    conv = jb.modules.DistributedConv2d(4, 4, 3, "cpu", (row, None), col, padding=1)
    soft = jb.modules.DistributedSoftmax(col, dim=-1)

    def tokens(x):          # (S / row, E / col)
        return soft(norm(lin(x)))

    xs = torch.randn(3, 5, 4, requires_grad=True)
    batched = torch.vmap(tokens)(xs)
    looped = torch.stack([tokens(x) for x in xs])
    assert_close(batched, looped, "vmap over linear -> layer norm -> softmax", 1e-5, 1e-6)
    gb = torch.autograd.grad(batched.square().sum(), [xs, lin.weight, norm.weight])
    gl = torch.autograd.grad(looped.square().sum(), [xs, lin.weight, norm.weight])
    for a, b, name in zip(gb, gl, ("input", "linear weight", "norm weight")):
        assert_close(a, b, f"vmap gradient of {name}", 1e-4, 1e-6)

    def image(x):           # (1, C / col, H / row, W)
        return conv(x)

    imgs = torch.randn(3, 1, 2, 6, 7, requires_grad=True)
    batched = torch.vmap(image)(imgs)
    looped = torch.stack([image(x) for x in imgs])
    assert_close(batched, looped, "vmap over a halo convolution", 1e-5, 1e-6)
    gb = torch.autograd.grad(batched.square().sum(), [imgs, conv.weight])
    gl = torch.autograd.grad(looped.square().sum(), [imgs, conv.weight])
    for a, b, name in zip(gb, gl, ("input", "conv weight")):
        assert_close(a, b, f"vmap gradient of {name}", 1e-4, 1e-6)


def test_vmap_over_distributed_layers():
    run_distributed(_worker_vmap, 4)
