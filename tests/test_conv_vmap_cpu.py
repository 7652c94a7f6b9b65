"""Convolutions and transposed convolutions under ``torch.vmap`` on a 2 x 2 mesh (width cut over the rows of the
mesh, channels over its columns), against a loop over the ensemble members.

Two ways of forming the ensemble: one layer applied to a stack of inputs, and a stack of the members' weights
run through ``functional_call`` (with the input stacked too, or shared by all members).  Three kinds of layer:
kernel equal to stride (nothing to fetch from neighbours), a 3 x 3 kernel with a halo, and grouped channels that
stay whole on a rank.  Gradients are taken by ordinary autograd through the batched forward.

Reference behaviours covered: tests/modules/convolution/test_conv_vmap.py (member weights with batched and shared
input, shared weights; forward, input gradient, weight gradients).
"""

import pytest
import torch

from dist_utils import assert_close, run_distributed, split

MEMBERS, CH, SIZE = 2, 4, 8
KINDS = {
    "no_halo": dict(kernel_size=2, stride=2),
    "halo": dict(kernel_size=3, stride=1, padding=1),
    "whole_groups": dict(kernel_size=2, stride=2, groups=2),
}


def _layer(transposed, kind, mesh, seed):
    import jigsaw_b200 as jb

    cls = jb.modules.DistributedConvTranspose2d if transposed else jb.modules.DistributedConv2d
    jb.launch.set_all_seeds(seed * 7 + mesh["col"].rank())                     # weight pieces differ over the channel ranks
    layer = cls(CH, CH, device="cpu", spatial_group=(None, mesh["row"]), channel_group=mesh["col"], bias=True, **KINDS[kind])
    jb.parallel.broadcast_replicas(layer)
    return layer


def _inputs(mesh):
    gen = torch.Generator().manual_seed(20)
    x = torch.randn(MEMBERS, 3, CH, SIZE, SIZE, generator=gen)
    return split(x, {2: mesh["col"], 4: mesh["row"]}).contiguous()


def _worker_member_weights(rank, world, transposed, kind, shared_input):
    import jigsaw_b200 as jb
    from torch.func import functional_call, stack_module_state

    mesh = jb.make_process_mesh({"row": 2, "col": 2})
    members = [_layer(transposed, kind, mesh, s) for s in range(MEMBERS)]
    base = _layer(transposed, kind, mesh, 99)
    params, buffers = stack_module_state(members)
    params = {k: v.detach().clone().requires_grad_(True) for k, v in params.items()}
    x = _inputs(mesh)
    x = (x[0] if shared_input else x).clone().requires_grad_(True)
    got = torch.vmap(lambda p, b, xi: functional_call(base, (p, b), (xi,)), in_dims=(0, 0, None if shared_input else 0))(
        params, buffers, x)
    want = torch.stack([m(x if shared_input else x[e]) for e, m in enumerate(members)])
    tag = f"{'transposed ' if transposed else ''}{kind}, {'shared' if shared_input else 'stacked'} input"
    assert_close(got, want, f"{tag}: output", 1e-4, 1e-5)
    weights = torch.randn(want.shape, generator=torch.Generator().manual_seed(5 + rank))
    (got * weights).sum().backward()
    gx, x.grad = x.grad.clone(), None
    (want * weights).sum().backward()
    assert_close(gx, x.grad, f"{tag}: input gradient", 1e-3, 1e-4)
    # functional_call hands the layer tensors without replica marks: sum over the tiles afterwards, as the members did
    named = dict(base.named_parameters())
    for n, p in params.items():
        jb.parallel.mark_replicated(p, jb.parallel.replica_groups(named[n]))
    jb.parallel.reduce_replica_grads(params.values())
    for n, p in params.items():
        want_grad = torch.stack([dict(m.named_parameters())[n].grad for m in members])
        assert_close(p.grad, want_grad, f"{tag}: gradient of {n}", 1e-3, 1e-4)


@pytest.mark.parametrize("shared_input", [False, True], ids=["stacked_input", "shared_input"])
@pytest.mark.parametrize("kind", list(KINDS))
@pytest.mark.parametrize("transposed", [False, True], ids=["conv", "conv_transpose"])
def test_stacked_member_weights(transposed, kind, shared_input):
    run_distributed(_worker_member_weights, 4, transposed, kind, shared_input, timeout=300)


def _worker_shared_weights(rank, world):
    import jigsaw_b200 as jb

    mesh = jb.make_process_mesh({"row": 2, "col": 2})
    for transposed in (False, True):
        for kind in KINDS:
            layer = _layer(transposed, kind, mesh, 3)
            x = _inputs(mesh).requires_grad_(True)
            got = torch.vmap(layer)(x)
            want = torch.stack([layer(xi) for xi in x])
            tag = f"{'transposed ' if transposed else ''}{kind}, one layer"
            assert_close(got, want, f"{tag}: output", 1e-4, 1e-5)
            weights = torch.randn(want.shape, generator=torch.Generator().manual_seed(6 + rank))
            grads = torch.autograd.grad((got * weights).sum(), [x, layer.weight, layer.bias])
            wants = torch.autograd.grad((want * weights).sum(), [x, layer.weight, layer.bias])
            for g, w, name in zip(grads, wants, ("input", "weight", "bias")):
                assert_close(g, w, f"{tag}: gradient of {name}", 1e-3, 1e-4)


def test_one_layer_over_stacked_inputs():
    run_distributed(_worker_shared_weights, 4, timeout=300)
