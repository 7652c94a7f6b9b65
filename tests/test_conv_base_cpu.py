"""Convolution layers outside the numeric parity tests: channel sizes after construction and re-sharding, configs
that survive a re-shard, argument validation (before any collective), patchify windows, parameter counts, the
conversion round trip reproducing the distributed forward, ``vmap`` over stacked weights.

Reference behaviours covered: tests/modules/convolution/conv/test_conv_base.py:30-91 (channel sizes, config),
:93-210 (argument validation), :213-277 (parameter counts), :279-332 (round trip), :334-372 (vmap over weights).
"""

import pytest
import torch

from dist_utils import assert_close, run_distributed, split


def _worker_conv_base(rank, world):
    import jigsaw_b200 as jb
    import torch.distributed as dist
    from jigsaw_b200.modules import convolution

    M = jb.modules
    m22 = jb.make_process_mesh({"row": 2, "col": 2})
    m14 = jb.make_process_mesh({"row": 1, "col": 4})
    world_group = dist.group.WORLD
    # channel sizes are global, like torch's; the shard is visible as local_out_channels
    conv = M.DistributedConv2d(8, 12, 2, "cpu", m22["row"], m22["col"], stride=2)
    assert (conv.in_channels, conv.out_channels) == (8, 12) and conv.local_out_channels == 6 == conv.weight.shape[0]
    conv.reshard_parameters(m22, m14)
    assert (conv.in_channels, conv.out_channels) == (8, 12) and conv.local_out_channels == 3 == conv.weight.shape[0]

    # a config subclass and its channel transport survive a re-shard
    class Config(convolution.ConvNdConfig):
        pass

    cfg = Config(m22["col"], None, (2, 2), (2, 2), "cpu", channel_comm="isend")
    conv = M.DistributedConv2d(8, 12, 2, "cpu", m22["row"], m22["col"], stride=2, bias=False, config=cfg)
    conv.reshard_parameters(m22, m14)
    assert type(conv.config) is Config and str(conv.config.channel_comm) == "isend"
    # argument validation, the same on every rank and before any collective
    for cin, cout in ((3, 4), (4, 3)):
        with pytest.raises(ValueError, match="channel group size"):
            M.DistributedConv2d(cin, cout, 3, "cpu", m22["row"], m22["col"])
    for arg in ("kernel_size", "stride", "padding", "dilation"):
        kwargs = {"kernel_size": 3, arg: (1, 1, 1)}
        with pytest.raises(ValueError, match="1 or 2 entries"):
            M.DistributedConv2d(24, 24, device="cpu", spatial_group=world_group, channel_group=world_group, **kwargs)
    for padding, stride in (("full", 1), ("same", 2)):
        with pytest.raises(ValueError, match="padding"):
            M.DistributedConv2d(24, 24, 3, "cpu", world_group, world_group, stride=stride, padding=padding)
    for groups in (1, 2):
        patch = M.DistributedConv1d(4, 4, 4, "cpu", m22["row"], m22["col"], stride=4, groups=groups)
        with pytest.raises(ValueError, match="multiple of"):
            patch(torch.randn(1, 2, 5))
    for mode in ("reflect", "replicate", "circular"):
        with pytest.raises(NotImplementedError, match="padding_mode"):
            M.DistributedConv2d.convert_to_jigsaw(torch.nn.Conv2d(8, 8, 3, padding=1, padding_mode=mode),
                                                  {"row": world_group, "col": world_group, "model": world_group}, "cpu")
    # padding="same": symmetric kernels work on a split; an asymmetric one is built where nothing is split and
    # refused, before the weights change, when a re-shard would put it onto a split
    same3 = M.DistributedConv2d(8, 12, 3, "cpu", m22["row"], m22["col"], padding="same")
    assert same3(torch.randn(1, 4, 6, 3)).shape == (1, 6, 6, 3)
    same4 = M.DistributedConv2d(8, 12, 4, "cpu", m14["row"], m14["col"], padding="same", groups=4)
    assert same4(torch.randn(1, 2, 6, 6)).shape == (1, 3, 6, 6)
    weight = same4.weight
    with pytest.raises(NotImplementedError, match="asymmetrically"):
        same4.reshard_parameters(m14, m22)
    assert same4.weight is weight
    # parameter counts are global and the same on every rank
    for nd, cls, ref in ((1, M.DistributedConv1d, torch.nn.Conv1d), (2, M.DistributedConv2d, torch.nn.Conv2d), (3, M.DistributedConv3d, torch.nn.Conv3d)):
        for bias in (True, False):
            want = sum(p.numel() for p in ref(8, 12, 3, bias=bias).parameters())
            assert cls(8, 12, 3, "cpu", m22["row"], m22["col"], padding=1, bias=bias).get_parameter_count() == want
            assert cls(8, 12, 3, "cpu", m14["row"], m14["col"], padding=1, bias=bias).get_parameter_count() == want
    # the conversion round trip reproduces the distributed forward
    torch.manual_seed(0)
    ref = torch.nn.Conv2d(8, 12, 3, padding=1).double()
    layer = M.DistributedConv2d.convert_to_jigsaw(ref, m22, "cpu")
    x = torch.randn(2, 8, 6, 8, dtype=torch.float64)
    cuts = {1: m22["col"], 3: m22["row"]}
    y = layer(split(x, cuts))
    assert_close(y, split(ref(x).detach(), cuts), "converted layer: forward", 1e-12, 1e-12)
    again = M.DistributedConv2d.convert_to_jigsaw(layer.convert_to_torch(m22), m22, "cpu")
    assert_close(again(split(x, cuts)), y.detach(), "round trip: forward", 0, 0)
    # vmap over stacked weights (an ensemble of kernels), without a bias
    layer = M.DistributedConv2d(4, 4, 3, "cpu", m22["row"], m22["col"], padding=1, bias=False, dtype=torch.float64)
    members = torch.stack([layer.weight.detach() * (i + 1) for i in range(3)])
    xl = torch.randn(1, 2, 6, 4, dtype=torch.float64)

    def one(w):
        return torch.func.functional_call(layer, {"weight": w}, (xl,))

    got = torch.vmap(one)(members)
    want = torch.stack([one(members[i]) for i in range(3)])
    assert_close(got, want, "vmap over stacked weights", 1e-12, 1e-12)


def test_conv_layer_contracts():
    run_distributed(_worker_conv_base, 4, timeout=300)
