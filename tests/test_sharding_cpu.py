"""Sweep of the four conversions (torch -> sharded, sharded -> torch, merge, re-shard) over layer kinds and meshes.

For linear layers and 1- / 2- / 3-D (transposed) convolutions, with and without bias: converting onto a mesh and
back returns the original parameters; merging returns the global tensors; re-sharding from mesh A to mesh B keeps
the values AND leaves a layer that computes exactly what a layer converted straight onto B computes (forward and
all gradients), which is what makes it safe to keep training on the new mesh.  Layer norm, group norm and roll
follow the same contract.

Reference behaviours covered: tests/test_sharding_configs.py:138-196 (round trips on 4 and 8 ranks), :198-245
(merge), :247-384 (values and functional equivalence after a re-shard), :386-425 (a model re-sharded layer by
layer), :427-444 (the grouped transposed case that is refused), :446-575 (norm layers), :577-621 (roll);
tests/test_param_count.py (parameter counts with replicas counted once).
"""

import copy

import torch

from dist_utils import all_ok, assert_close, run_distributed, split

KINDS = ("linear", "conv1d", "conv2d", "conv3d", "convT1d", "convT2d", "convT3d")


def _make_torch(kind, bias):
    torch.manual_seed(1234)                                   # every rank builds the same reference
    k = 3
    return {"linear": lambda: torch.nn.Linear(24, 16, bias=bias),
            "conv1d": lambda: torch.nn.Conv1d(24, 16, k, stride=k, bias=bias),
            "conv2d": lambda: torch.nn.Conv2d(24, 16, k, stride=k, bias=bias),
            "conv3d": lambda: torch.nn.Conv3d(24, 16, k, stride=k, bias=bias),
            "convT1d": lambda: torch.nn.ConvTranspose1d(24, 16, k, stride=k, bias=bias),
            "convT2d": lambda: torch.nn.ConvTranspose2d(24, 16, k, stride=k, bias=bias),
            "convT3d": lambda: torch.nn.ConvTranspose3d(24, 16, k, stride=k, bias=bias)}[kind]().double()


def _meshes4():
    import jigsaw_b200 as jb

    mp = ("row", "col")
    return {"2x2": jb.make_process_mesh({"row": 2, "col": 2}), "4x1": jb.make_process_mesh({"row": 4, "col": 1}),
            "1x4": jb.make_process_mesh({"row": 1, "col": 4}),
            "2x1x2": jb.make_process_mesh({"dp": 2, "row": 1, "col": 2}, model_parallel_axes=mp),
            "2x2x1": jb.make_process_mesh({"dp": 2, "row": 2, "col": 1}, model_parallel_axes=mp),
            "4x1x1": jb.make_process_mesh({"dp": 4, "row": 1, "col": 1}, model_parallel_axes=mp)}


PAIRS = [("2x2", "2x2"), ("4x1", "1x4"), ("1x4", "4x1"), ("2x2", "4x1x1"), ("4x1x1", "2x2"), ("2x2", "2x1x2"),
         ("2x2x1", "2x2"), ("2x1x2", "2x2x1"), ("1x4", "2x1x2"), ("4x1", "2x2x1"), ("2x2", "1x4")]


def _local_input(layer, kind):
    torch.manual_seed(99)
    if kind == "linear":
        return torch.randn(2, 8, layer.weight.shape[1], dtype=torch.float64)
    n = int(kind[-2])
    spatial = [12] * n
    last = layer.spatial_groups[-1]
    spatial[-1] //= 1 if last is None else last.size()
    return torch.randn(2, layer.in_channels // layer.channel_group.size(), *spatial, dtype=torch.float64)


def _fwd_bwd(layer, x):
    x = x.detach().clone().requires_grad_(True)
    layer.zero_grad(set_to_none=True)
    y = layer(x)
    torch.manual_seed(7)
    y.backward(torch.randn_like(y))
    return y.detach(), x.grad, [None if p.grad is None else p.grad.clone() for p in layer.parameters()]


def _params_equal(a, b, what):
    assert_close(a.weight.data, b.weight.data, f"{what}: weight", 0, 0)
    assert all_ok((a.bias is None) == (b.bias is None)), f"{what}: bias presence"
    if b.bias is not None:
        assert_close(a.bias.data, b.bias.data, f"{what}: bias", 0, 0)


def _worker_sweep(rank, world):
    from jigsaw_b200 import convert

    meshes = _meshes4()
    for kind in KINDS:
        for bias in (True, False):
            ref = _make_torch(kind, bias)
            # round trip and merge on every mesh
            for name, mesh in meshes.items():
                if not bias and name != "2x2":
                    continue
                layer = convert.convert_to_jigsaw(copy.deepcopy(ref), mesh, "cpu")
                _params_equal(layer.convert_to_torch(mesh), ref, f"{kind} on {name}: round trip")
                w, b = layer.merge_weights(mesh)
                assert_close(w, ref.weight.data, f"{kind} on {name}: merged weight", 0, 0)
                assert all_ok((b is None) == (not bias))
            # re-shard: values survive, and the layer equals one converted straight onto the target mesh
            for src, dst in (PAIRS if bias else PAIRS[:1]):
                moved = convert.convert_to_jigsaw(copy.deepcopy(ref), meshes[src], "cpu")
                moved.reshard_parameters(meshes[src], meshes[dst])
                _params_equal(moved.convert_to_torch(meshes[dst]), ref, f"{kind} {src} -> {dst}: values")
                direct = convert.convert_to_jigsaw(copy.deepcopy(ref), meshes[dst], "cpu")
                x = _local_input(direct, kind)
                y1, dx1, g1 = _fwd_bwd(moved, x)
                y2, dx2, g2 = _fwd_bwd(direct, x)
                tag = f"{kind} {src} -> {dst}"
                assert_close(y1, y2, f"{tag}: forward", 0, 0)
                assert_close(dx1, dx2, f"{tag}: input gradient", 0, 0)
                for a, b2 in zip(g1, g2):
                    assert_close(a, b2, f"{tag}: parameter gradient", 0, 0)


def test_round_trips_merges_and_reshards_on_four_ranks():
    run_distributed(_worker_sweep, 4, timeout=900)


def _worker_eight(rank, world):
    """Round trips on the two 8-rank layouts, norm layers and roll across meshes, a model moved layer by layer,
    parameter counts with replicas counted once."""
    import jigsaw_b200 as jb
    from jigsaw_b200 import convert

    M = jb.modules
    m42 = jb.make_process_mesh({"row": 4, "col": 2})
    m24 = jb.make_process_mesh({"row": 2, "col": 4})
    for kind in KINDS:
        ref = _make_torch(kind, True)
        for name, mesh in (("4x2", m42), ("2x4", m24)):
            layer = convert.convert_to_jigsaw(copy.deepcopy(ref), mesh, "cpu")
            _params_equal(layer.convert_to_torch(mesh), ref, f"{kind} on {name}: round trip")
            w, b = layer.merge_weights(mesh)
            assert_close(w, ref.weight.data, f"{kind} on {name}: merged weight", 0, 0)
        layer = convert.convert_to_jigsaw(copy.deepcopy(ref), m42, "cpu")
        layer.reshard_parameters(m42, m24)
        _params_equal(layer.convert_to_torch(m24), ref, f"{kind} 4x2 -> 2x4: values")
    # layer norm: values, round trip and re-shard (affine and not)
    for affine in (True, False):
        torch.manual_seed(5)
        ref = torch.nn.LayerNorm(16, elementwise_affine=affine).double()
        if affine:
            with torch.no_grad():
                ref.weight.copy_(torch.randn(16))
                ref.bias.copy_(torch.randn(16))
        ln = convert.convert_to_jigsaw(copy.deepcopy(ref), m42, "cpu")
        assert isinstance(ln, M.DistributedLayerNorm)
        ln.reshard_parameters(m42, m24)
        back = ln.convert_to_torch(m24)
        assert all_ok((back.weight is None) == (not affine))
        if affine:
            _params_equal(back, ref, "layer norm 4x2 -> 2x4")
        x = torch.randn(2, 8, 16, dtype=torch.float64)
        cuts = {1: m24["row"], 2: m24["col"]}
        assert_close(ln(split(x, cuts)), split(ref(x).detach(), cuts), "layer norm after the re-shard: output", 1e-10, 1e-10)
    # group norm: channels move between channel groups of different sizes
    gn = M.DistributedGroupNorm(4, 16, "cpu", channel_group=m42["col"], dtype=torch.float64)
    with torch.no_grad():                                     # a different value in every channel of every shard
        gn.weight.copy_(torch.arange(8, dtype=torch.float64) + 100 * m42["col"].rank())
        gn.bias.copy_(-torch.arange(8, dtype=torch.float64) - 100 * m42["col"].rank())
    w0, b0 = gn.merge_weights(m42)
    assert w0.shape == (16,) and float(w0[8]) == 100.0
    gn.reshard_parameters(m42, m24)
    w1, b1 = gn.merge_weights(m24)
    assert_close(w1, w0, "group norm 4x2 -> 2x4: weight", 0, 0)
    assert_close(b1, b0, "group norm 4x2 -> 2x4: bias", 0, 0)
    assert gn.weight.shape[0] == 16 // 4
    # a model moved layer by layer keeps computing the same function
    torch.manual_seed(8)
    serial = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.GELU(), torch.nn.LayerNorm(32), torch.nn.Linear(32, 16)).double()
    model = convert.convert_to_jigsaw(copy.deepcopy(serial), m42, "cpu")
    assert jb.debug.count_parameters(model, m42) == sum(p.numel() for p in serial.parameters())
    assert sum(m.get_parameter_count() for m in model if hasattr(m, "get_parameter_count")) == sum(p.numel() for p in serial.parameters())
    for layer in model:
        if hasattr(layer, "reshard_parameters"):
            layer.reshard_parameters(m42, m24)
    assert jb.debug.count_parameters(model, m24) == sum(p.numel() for p in serial.parameters())
    x = torch.randn(2, 8, 16, dtype=torch.float64)
    cuts = {1: m24["row"], 2: m24["col"]}
    assert_close(model(split(x, cuts)), split(serial(x).detach(), cuts), "model after a layer-by-layer re-shard", 1e-10, 1e-10)
    # roll: conversion with an explicit dimension map, then re-sharding onto other groups
    roll = M.Roll((2, -3), (1, 2), dtype=torch.float64)
    droll = convert.convert_to_jigsaw(roll, m42, "cpu", dim_to_mesh_axis={1: "row", 2: "col"})
    assert isinstance(droll, M.DistributedRoll)
    t = torch.arange(2 * 8 * 8, dtype=torch.float64).view(2, 8, 8)
    want = torch.roll(t, (2, -3), (1, 2))
    assert_close(droll(split(t, {1: m42["row"], 2: m42["col"]})), split(want, {1: m42["row"], 2: m42["col"]}), "roll on 4x2", 0, 0)
    droll.reshard((1, 2), (m24["row"], m24["col"]))
    assert_close(droll(split(t, {1: m24["row"], 2: m24["col"]})), split(want, {1: m24["row"], 2: m24["col"]}), "roll on 2x4", 0, 0)


def test_eight_rank_layouts_norms_model_and_roll():
    run_distributed(_worker_eight, 8, timeout=900)
