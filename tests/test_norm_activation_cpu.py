"""Layer norm conversion details (``eps``, ``bias`` flag, dtype and parameter names survive the round trip; forward and
gradients match torch for every affine / bias combination), group norm with and without a spatial split, softmax and
log-softmax with and without a group and under ``vmap`` with the batch dimension anywhere.

Reference behaviours covered: tests/modules/normalization/test_normalization.py:150-219 (round trip of eps, bias,
dtype), tests/modules/normalization/test_group_norm.py:30-46 and :117-179 (unsharded and spatially sharded group
norm), tests/modules/activation/test_activation.py (no group, sharded softmax), test_activation_vmap.py (vmap).
"""

import torch

from dist_utils import all_ok, assert_close, run_distributed, split


def _worker_norms(rank, world):
    import jigsaw_b200 as jb

    M = jb.modules
    mesh = jb.make_process_mesh({"row": 2, "col": 2})
    row, col, model = mesh["row"], mesh["col"], mesh["model"]
    for affine, bias in ((True, True), (True, False), (False, True)):
        ref = torch.nn.LayerNorm(8, eps=1e-2, elementwise_affine=affine, bias=bias, dtype=torch.float64)
        torch.manual_seed(0)
        if affine:
            with torch.no_grad():
                ref.weight.uniform_(0.5, 2.0)
                if bias:
                    ref.bias.uniform_(-1.0, 1.0)
        x = torch.randn(3, 5, 8, dtype=torch.float64)
        layer = M.DistributedLayerNorm.convert_to_jigsaw(ref, mesh, "cpu")
        tag = f"layer norm affine={affine} bias={bias}"
        assert all_ok(layer.eps == 1e-2 and layer.state_dict().keys() == ref.state_dict().keys()), f"{tag}: eps / names"
        assert all(p.dtype == torch.float64 for p in layer.parameters())
        xl = split(x, {2: col}).requires_grad_(True)
        xr = x.clone().requires_grad_(True)
        y, yr = layer(xl), ref(xr)
        y.sum().backward()
        yr.sum().backward()
        assert_close(y, split(yr.detach(), {2: col}), f"{tag}: forward", 1e-10, 1e-10)
        assert_close(xl.grad, split(xr.grad, {2: col}), f"{tag}: input gradient", 1e-10, 1e-10)
        back = layer.convert_to_torch(mesh)
        same = back.eps == 1e-2 and back.state_dict().keys() == ref.state_dict().keys() and all(
            torch.equal(back.state_dict()[k], v) for k, v in ref.state_dict().items())
        assert all_ok(same), f"{tag}: round trip"
    # group norm: without a spatial split it is torch's own kernel per shard; with one the statistics are shared
    torch.manual_seed(1)
    ref = torch.nn.GroupNorm(4, 8, eps=1e-3).double()
    with torch.no_grad():
        ref.weight.uniform_(0.5, 2.0)
        ref.bias.uniform_(-1.0, 1.0)
    x = torch.randn(2, 8, 6, 4, dtype=torch.float64)
    for spatial, cuts in ((None, {1: col}), ((row, None), {1: col, 2: row}), ((None, row), {1: col, 3: row})):
        gn = M.DistributedGroupNorm(4, 8, "cpu", channel_group=col, eps=1e-3, dtype=torch.float64, spatial_group=spatial)
        with torch.no_grad():
            gn.weight.copy_(split(ref.weight.data, {0: col}))
            gn.bias.copy_(split(ref.bias.data, {0: col}))
        xl = split(x, cuts).requires_grad_(True)
        xr = x.clone().requires_grad_(True)
        y, yr = gn(xl), ref(xr)
        g = torch.randn(yr.shape, generator=torch.Generator().manual_seed(2), dtype=torch.float64)
        y.backward(split(g, cuts))
        yr.backward(g)
        tag = f"group norm spatial={'none' if spatial is None else [None if s is None else s.size() for s in spatial]}"
        assert_close(y, split(yr.detach(), cuts), f"{tag}: forward", 1e-10, 1e-10)
        assert_close(xl.grad, split(xr.grad, cuts), f"{tag}: input gradient", 1e-10, 1e-10)
        ref.zero_grad()
    # softmax / log-softmax: without a group they are torch's, with one they match torch on the gathered tensor
    t = torch.randn(3, 4, 8, dtype=torch.float64)
    Fn = M.functional
    assert torch.equal(M.DistributedSoftmax(None, dim=1)(t), torch.softmax(t, 1))
    assert torch.equal(Fn.distributed_log_softmax(t, 1, None), torch.log_softmax(t, 1))
    for dim in (-1, 1):
        cuts = {dim % 3: col}
        sm = M.DistributedSoftmax(col, dim=dim)
        assert sm.get_parameter_count() == 0
        tl = split(t, cuts).requires_grad_(True)
        tr = t.clone().requires_grad_(True)
        y, yr = sm(tl), torch.softmax(tr, dim)
        g = torch.randn(t.shape, generator=torch.Generator().manual_seed(3), dtype=torch.float64)
        y.backward(split(g, cuts))
        yr.backward(g)
        assert_close(y, split(yr.detach(), cuts), f"softmax dim={dim}", 1e-12, 1e-12)
        assert_close(tl.grad, split(tr.grad, cuts), f"softmax dim={dim}: gradient", 1e-12, 1e-12)
        assert_close(Fn.distributed_log_softmax(split(t, cuts), dim, col), split(torch.log_softmax(t, dim), cuts), f"log-softmax dim={dim}", 1e-12, 1e-12)
        # vmap: batch dimension in front, and away from the front
        batched = torch.randn(5, 3, 4, 4, dtype=torch.float64)
        loop = torch.stack([sm(batched[i]) for i in range(5)])
        assert_close(torch.vmap(sm)(batched), loop, f"softmax dim={dim}: vmap", 1e-12, 1e-12)
        assert_close(torch.vmap(sm, in_dims=1)(batched.movedim(0, 1)), loop, f"softmax dim={dim}: vmap in_dims=1", 1e-12, 1e-12)


def test_norms_and_softmax_details():
    run_distributed(_worker_norms, 4, timeout=300)


def _worker_norm_vmap(rank, world):
    """Layer norm and softmax under ``vmap`` with the ensemble axis anywhere in the input, with and without affine
    parameters, and with stacked member weights (reference: tests/modules/normalization/test_normalization_vmap.py,
    tests/modules/activation/test_activation_vmap.py)."""
    import jigsaw_b200 as jb
    from torch.func import functional_call, stack_module_state

    mesh = jb.make_process_mesh({"row": 2, "col": 2})
    M, row, col = jb.modules, mesh["row"], mesh["col"]
    gen = torch.Generator().manual_seed(11 + rank)
    x = torch.randn(3, 2, 4, 8, generator=gen, dtype=torch.float64)                   # (members, batch, tokens / row, features / col)
    for affine in (True, False):
        jb.launch.set_all_seeds(5)
        ln = M.DistributedLayerNorm(16, mesh["model"].rank(), "cpu", row, col, elementwise_affine=affine, dtype=torch.float64)
        for in_dim in (0, 1, 2):
            moved = x.movedim(0, in_dim).contiguous().requires_grad_(True)
            got = torch.vmap(ln, in_dims=in_dim, out_dims=in_dim)(moved)
            want = torch.stack([ln(m) for m in moved.unbind(in_dim)], dim=in_dim)
            assert_close(got, want, f"layer norm affine={affine}, ensemble axis {in_dim}", 1e-12, 1e-12)
            seed = torch.randn(want.shape, generator=torch.Generator().manual_seed(3), dtype=torch.float64)
            (g,) = torch.autograd.grad(got, moved, seed, retain_graph=True)
            (w,) = torch.autograd.grad(want, moved, seed)
            assert_close(g, w, f"layer norm affine={affine}, ensemble axis {in_dim}: input gradient", 1e-10, 1e-12)
        assert ln.get_parameter_count() == (32 if affine else 0)
    members = []
    for s in range(3):
        jb.launch.set_all_seeds(20 + s)
        m = M.DistributedLayerNorm(16, mesh["model"].rank(), "cpu", row, col, dtype=torch.float64)
        with torch.no_grad():
            for p in m.parameters():
                p.add_(0.1 * torch.randn(p.shape, dtype=torch.float64))
        jb.parallel.broadcast_replicas(m)
        members.append(m)
    params, buffers = stack_module_state(members)
    got = torch.vmap(lambda p, b, xi: functional_call(members[0], (p, b), (xi,)))(params, buffers, x)
    assert_close(got, torch.stack([m(xi) for m, xi in zip(members, x)]), "layer norm with member weights", 1e-12, 1e-12)
    soft = M.DistributedSoftmax(col, dim=-1)
    for in_dim in (0, 2):
        moved = x.movedim(0, in_dim).contiguous()
        got = torch.vmap(soft, in_dims=in_dim, out_dims=in_dim)(moved)
        assert_close(got, torch.stack([soft(m) for m in moved.unbind(in_dim)], dim=in_dim), f"softmax, ensemble axis {in_dim}", 1e-12, 1e-12)


def test_layer_norm_and_softmax_under_vmap_with_the_ensemble_axis_anywhere():
    run_distributed(_worker_norm_vmap, 4, timeout=300)
