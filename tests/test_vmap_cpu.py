"""``torch.vmap`` over the distributed layers (ensembles of inputs): the batched call must equal a
loop over the ensemble members, forward and gradients."""

import torch

from dist_utils import assert_close, run_distributed, split


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


def _worker_ensemble(rank, world):
    """An ensemble as stacked weights: ``torch.vmap`` over ``functional_call`` with the members' parameters
    stacked along a new first axis.  Outputs equal the members run one by one; ``functional_call`` hands the
    layers tensors without replica marks, so the gradients of replicated parameters are summed afterwards
    with ``reduce_replica_grads`` (marks copied from a member)."""
    import jigsaw_b200 as jb
    from torch.func import functional_call, stack_module_state

    mesh = jb.make_process_mesh({"row": 2, "col": 2})
    row, col, model = mesh["row"], mesh["col"], mesh["model"]

    def member(seed):
        jb.launch.set_all_seeds(seed * 10 + model.rank())
        net = torch.nn.Sequential(jb.modules.DistributedLinear(8, 8, "cpu", model, row, col),
                                  jb.modules.DistributedLayerNorm(8, model.rank(), "cpu", row, col))
        with torch.no_grad():
            for p in net[1].parameters():
                p.add_(torch.randn_like(p) * 0.1)
        jb.parallel.broadcast_replicas(net)
        return net

    members = [member(s) for s in range(3)]
    torch.manual_seed(0)
    x = split(torch.randn(6, 8), {0: row, 1: col})
    g = split(torch.randn(6, 8), {0: row, 1: col})
    outs, grads = [], []
    for net in members:
        y = net(x)
        (y * g).sum().backward()
        outs.append(y.detach())
        grads.append({n: p.grad.clone() for n, p in net.named_parameters()})
    params, buffers = stack_module_state(members)
    params = {k: v.detach().clone().requires_grad_(True) for k, v in params.items()}
    base = members[0]
    y = torch.vmap(lambda p, b: functional_call(base, (p, b), (x,)), in_dims=(0, 0))(params, buffers)
    assert_close(y.detach(), torch.stack(outs), "ensemble output", 1e-5, 1e-6)
    (y * g).sum().backward()
    named = dict(base.named_parameters())
    for n, p in params.items():
        groups = jb.parallel.replica_groups(named[n])
        if groups:
            jb.parallel.mark_replicated(p, groups)
    jb.parallel.reduce_replica_grads(params.values())
    for n, p in params.items():
        assert_close(p.grad, torch.stack([gr[n] for gr in grads]), f"ensemble gradient of {n}", 1e-4, 1e-5)


def test_ensemble_of_stacked_weights():
    run_distributed(_worker_ensemble, 4)


def _worker_nested_vmap(rank, world):
    """The rules re-apply their Function to the stack, so nested ``vmap`` levels unwind one after the other:
    two levels over a gather, a sum and a sharded linear layer equal the double loop."""
    import jigsaw_b200 as jb
    from jigsaw_b200._core.collectives import all_gather_cat, all_reduce_sum

    mesh = jb.make_process_mesh({"row": 2, "col": 2})
    row, col = mesh["row"], mesh["col"]
    x = torch.arange(2 * 3 * 4, dtype=torch.float64).view(2, 3, 4) + 100 * rank
    for name, fn in (("gather", lambda t: all_gather_cat(t, row, 0)), ("sum", lambda t: all_reduce_sum(t, col))):
        got = torch.vmap(torch.vmap(fn))(x)
        want = torch.stack([torch.stack([fn(x[i, j]) for j in range(3)]) for i in range(2)])
        assert_close(got, want, f"nested vmap over {name}", 0, 0)
    torch.manual_seed(0)
    lin = jb.modules.DistributedLinear(8, 12, "cpu", mesh["model"], row, col, dtype=torch.float64)
    tokens = torch.randn(2, 3, 4, 4, dtype=torch.float64)            # (outer, inner, tokens / row, features / col)
    got = torch.vmap(torch.vmap(lin))(tokens)
    want = torch.stack([torch.stack([lin(tokens[i, j]) for j in range(3)]) for i in range(2)])
    assert_close(got, want, "nested vmap over a sharded linear layer", 1e-12, 1e-12)


def test_nested_vmap():
    run_distributed(_worker_nested_vmap, 4)


def _worker_linear_members_nested(rank, world):
    """Member weights at one ``vmap`` level and the input at another, in both orders, and member weights at both
    levels (a grid of members): each equals the loops over the same members and inputs."""
    import jigsaw_b200 as jb
    from torch.func import functional_call, stack_module_state

    mesh = jb.make_process_mesh({"row": 2, "col": 2})
    row, col, model = mesh["row"], mesh["col"], mesh["model"]
    E, B = 3, 2

    def layer(seed):
        jb.launch.set_all_seeds(seed * 13 + model.rank())
        lin = jb.modules.DistributedLinear(8, 12, "cpu", model, row, col)
        jb.parallel.broadcast_replicas(lin)
        return lin

    members = [layer(s) for s in range(E)]
    base = layer(50)
    params, _ = stack_module_state(members)
    params = {k: v.detach().clone().requires_grad_(True) for k, v in params.items()}
    x = torch.randn(E, B, 2, 5, 4, generator=torch.Generator().manual_seed(rank))

    def call(p, xi):
        return functional_call(base, p, (xi,))

    want = torch.stack([torch.stack([m(xi) for xi in x[e]]) for e, m in enumerate(members)])
    got = torch.vmap(lambda p, xe: torch.vmap(lambda xi: call(p, xi))(xe))(params, x)
    assert_close(got, want, "members outside, inputs inside", 1e-5, 1e-6)
    g = torch.randn(want.shape, generator=torch.Generator().manual_seed(9 + rank))
    (got * g).sum().backward()
    (want * g).sum().backward()
    named = dict(base.named_parameters())
    for n, p in params.items():
        jb.parallel.mark_replicated(p, jb.parallel.replica_groups(named[n]))
    jb.parallel.reduce_replica_grads(params.values())
    for n, p in params.items():
        assert_close(p.grad, torch.stack([dict(m.named_parameters())[n].grad for m in members]), f"gradient of {n}", 1e-4, 1e-5)
    # inputs outside, members inside
    got = torch.vmap(lambda xb: torch.vmap(call)(params, xb))(x.transpose(0, 1))
    assert_close(got, want.transpose(0, 1), "inputs outside, members inside", 1e-5, 1e-6)
    # a grid of members: weights batched at both levels
    grid = {k: torch.stack([v.detach(), 2 * v.detach()], 1) for k, v in params.items()}          # (E, 2, ...)
    got = torch.vmap(torch.vmap(call))(grid, x)
    scaled = torch.stack([want[:, 0], 2 * torch.stack([m(x[e, 1]) for e, m in enumerate(members)])], 1)
    assert_close(got, scaled, "members at both levels", 1e-5, 1e-6)


def test_linear_member_weights_at_either_vmap_level():
    run_distributed(_worker_linear_members_nested, 4)
