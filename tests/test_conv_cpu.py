"""Distributed convolutions on CPU/gloo ranks against the undivided torch layers:
output, input gradient and every parameter gradient, over several meshes, strides,
dilations, channel strategies and the transposed variants."""

import pytest
import torch

from dist_utils import assert_close, run_distributed, split


def _conv_case(mesh, nd, cin, cout, k, s, p, d, groups, transposed, channel_comm, size, seed):
    import jigsaw_b200 as jb

    torch.manual_seed(seed)
    M = jb.modules
    axes = ["sd", "sh", "sw"][3 - nd:]
    sgroups = [mesh[a] for a in axes]
    col = mesh["col"]
    torch_cls = {(1, False): torch.nn.Conv1d, (2, False): torch.nn.Conv2d, (3, False): torch.nn.Conv3d,
                 (1, True): torch.nn.ConvTranspose1d, (2, True): torch.nn.ConvTranspose2d, (3, True): torch.nn.ConvTranspose3d}[(nd, transposed)]
    dist_cls = {(1, False): M.DistributedConv1d, (2, False): M.DistributedConv2d, (3, False): M.DistributedConv3d,
                (1, True): M.DistributedConvTranspose1d, (2, True): M.DistributedConvTranspose2d, (3, True): M.DistributedConvTranspose3d}[(nd, transposed)]
    ref = torch_cls(cin, cout, k, stride=s, padding=p, dilation=d, groups=groups).double()
    layer = dist_cls(cin, cout, k, "cpu", sgroups, col, stride=s, padding=p, dilation=d, groups=groups,
                     dtype=torch.float64, channel_comm=channel_comm)
    layer._load_global(ref.weight.data, ref.bias.data)
    x = torch.randn(2, cin, *size, dtype=torch.float64)
    x_ref = x.clone().requires_grad_(True)
    y_ref = ref(x_ref)
    gy = torch.randn_like(y_ref)
    y_ref.backward(gy)
    in_spec = {1: col, **{2 + i: g for i, g in enumerate(sgroups)}}
    xl = split(x, in_spec).requires_grad_(True)
    y = layer(xl)
    tag = f"nd={nd} T={transposed} k={k} s={s} p={p} d={d} g={groups} cc={channel_comm}"
    assert_close(y, split(y_ref.detach(), in_spec), f"output {tag}", 1e-9, 1e-9)
    y.backward(split(gy, in_spec))
    assert_close(xl.grad, split(x_ref.grad, in_spec), f"dx {tag}", 1e-9, 1e-9)
    wdim = layer._weight_shard_dim
    assert_close(layer.weight.grad, split(ref.weight.grad, {wdim: col}), f"dW {tag}", 1e-9, 1e-9)
    assert_close(layer.bias.grad, split(ref.bias.grad, {0: col}), f"db {tag}", 1e-9, 1e-9)
    # round trip through merge / convert_to_torch
    back = layer.convert_to_torch({"col": col, "row": sgroups[-1]})
    assert_close(back.weight.data, ref.weight.data, f"merge {tag}", 0, 0)


def _worker_2d(rank, world):
    import jigsaw_b200 as jb

    mesh = jb.make_process_mesh({"sh": 2, "sw": 2, "col": 1})
    mesh["sd"] = None
    for (k, s, p, d) in [(3, 1, 1, 1), (5, 1, 2, 1), (3, 2, 1, 1), (3, 1, 2, 2), (4, 4, 0, 1), (2, 2, 0, 1)]:
        _conv_case(mesh, 2, 4, 6, k, s, p, d, 1, False, "auto", (16, 24), 0)
    for (k, s, p) in [(2, 2, 0), (4, 2, 1), (3, 1, 1)]:
        _conv_case(mesh, 2, 4, 6, k, s, p, 1, 1, True, "auto", (8, 12), 1)
    # parameters were marked and identical across the spatial groups
    layer = jb.modules.DistributedConv2d(3, 5, 3, "cpu", (mesh["sh"], mesh["sw"]), mesh["col"], padding=1)
    assert len(jb.parallel.replica_groups(layer.weight)) == 2
    jb.debug.assert_replica_consistency(layer, {"sh": mesh["sh"], "sw": mesh["sw"]})
    assert "spatial=(2, 2), channel=1" in repr(layer)
    assert layer.get_parameter_count() == 5 * 3 * 9 + 5


def _worker_channels(rank, world):
    import jigsaw_b200 as jb

    mesh = jb.make_process_mesh({"sw": 2, "col": 2})
    mesh["sd"] = mesh["sh"] = None
    for cc in ("all_gather", "batch_isend_irecv", "isend"):
        _conv_case(mesh, 2, 4, 8, 3, 1, 1, 1, 1, False, cc, (8, 16), 2)
        _conv_case(mesh, 2, 4, 8, 4, 2, 1, 1, 1, True, cc, (6, 8), 3)
        _conv_case(mesh, 1, 4, 8, 3, 1, 1, 1, 1, False, cc, (16,), 4)
    _conv_case(mesh, 2, 4, 8, 3, 1, 1, 1, 2, False, "auto", (8, 16), 5)     # channel-local groups
    _conv_case(mesh, 2, 8, 4, 2, 2, 0, 1, 2, True, "auto", (6, 8), 6)


def _worker_3d(rank, world):
    import jigsaw_b200 as jb

    mesh = jb.make_process_mesh({"sd": 2, "sh": 2, "sw": 2, "col": 1})
    _conv_case(mesh, 3, 2, 4, 3, 1, 1, 1, 1, False, "auto", (8, 8, 8), 7)
    _conv_case(mesh, 3, 2, 4, 3, 2, 1, 1, 1, False, "auto", (8, 8, 8), 8)
    _conv_case(mesh, 3, 4, 2, 4, 2, 1, 1, 1, True, "auto", (4, 4, 4), 9)


def _worker_errors(rank, world):
    import jigsaw_b200 as jb

    mesh = jb.make_process_mesh({"sw": 2, "col": 1})
    M = jb.modules
    with pytest.raises(NotImplementedError):
        M.DistributedConv2d(2, 2, 4, "cpu", mesh["sw"], mesh["col"], padding="same")
    with pytest.raises(ValueError):
        M.DistributedConv2d(3, 4, 3, "cpu", mesh["sw"], mesh["col"], groups=2)
    with pytest.raises(NotImplementedError):
        M.DistributedConvTranspose2d(2, 2, 3, "cpu", mesh["sw"], mesh["col"], output_padding=1)
    layer = M.DistributedConv2d(2, 2, 3, "cpu", mesh["sw"], mesh["col"], stride=2, padding=0)
    with pytest.raises(NotImplementedError):     # global output not divisible by the group
        layer(torch.randn(1, 2, 8, 6))
    with pytest.raises(ValueError):
        layer(torch.randn(2, 8))
    # unbatched input
    layer = M.DistributedConv2d(2, 3, 3, "cpu", mesh["sw"], mesh["col"], padding=1)
    assert layer(torch.randn(2, 8, 6)).shape == (3, 8, 6)
    # config built for another layer is rejected
    cfg = M.ConvNdConfig(mesh["col"], None, (3, 3), (1, 1), "cpu")
    with pytest.raises(ValueError):
        M.DistributedConv2d(2, 3, 3, "cpu", mesh["sw"], mesh["col"], padding=1, config=cfg)


def test_conv2d_spatial_2x2():
    run_distributed(_worker_2d, 4)


def test_conv_channel_parallel():
    run_distributed(_worker_channels, 4)


def test_conv3d_2x2x2():
    run_distributed(_worker_3d, 8)


def test_conv_errors():
    run_distributed(_worker_errors, 2)


def _worker_sweep_1d(rank, world, transposed, k):
    """Span arithmetic under a 4-way split: every (stride, padding, dilation) combination of a small grid that
    the layer accepts for this kernel size must match the undivided layer exactly (float64)."""
    import jigsaw_b200 as jb

    mesh = jb.make_process_mesh({"sw": 4, "col": 1})
    mesh["sd"] = mesh["sh"] = None
    accepted = 0
    for s in (1, 2, 3):
        for p in (0, 1, 2):
            for d in (1, 2):
                if transposed and (d > 1 or p > (k - 1)):
                    continue
                try:
                    _conv_case(mesh, 1, 2, 3, k, s, p, d, 1, transposed, "auto", (48,), k * 100 + s * 10 + p)
                    accepted += 1
                except (ValueError, NotImplementedError) as e:     # geometry the layer rejects, on every rank alike
                    assert "AssertionError" not in type(e).__name__
    assert accepted >= (1 if transposed else 3), accepted


@pytest.mark.parametrize("k", [1, 2, 3, 4, 5])
@pytest.mark.parametrize("transposed", [False, True], ids=["conv", "conv_transpose"])
def test_conv1d_parameter_sweep_four_ranks(transposed, k):
    run_distributed(_worker_sweep_1d, 4, transposed, k, timeout=600)
