"""The parts under the convolution layers, each on its own: how constructor arguments are normalised, how the
channel options resolve, and the two halo operations as linear maps.

``span_gather`` builds, from the tiles of an axis, the span a rank's outputs read (zeros outside the domain);
``span_reduce`` adds the overhang of a rank's raw transposed-convolution output into its neighbours.  Each is the
other's adjoint, which is what makes them each other's backward pass; that is checked as <gather(x), y> =
<x, reduce(y)> summed over the ranks, besides the comparison with padded convolutions of the undivided tensor.

Reference behaviours covered: tests/modules/convolution/common/test_arg_norm.py, test_channel_comm.py (option
resolution and group validation), test_halo_singleton.py (gather / reduce against padded convolutions and as
adjoints), test_layer_inputs.py (inputs of the wrong rank, configurations of another layer).
"""

import pytest
import torch

from dist_utils import all_ok, assert_close, run_distributed, split
from jigsaw_b200.modules.convolution import _args


def test_sizes_are_broadcast_per_axis():
    assert _args.ntuple(3, 2) == (3, 3) and _args.ntuple((3,), 3) == (3, 3, 3) and _args.ntuple([1, 2], 2) == (1, 2)
    for bad in ((1, 2, 3), ()):
        with pytest.raises(ValueError, match="one per spatial axis"):
            _args.ntuple(bad, 2)


def test_padding_names():
    assert _args.resolve_padding("valid", (3, 3), (1, 1), (1, 1)) == (0, 0)
    assert _args.resolve_padding("same", (3, 5), (1, 1), (1, 2)) == (1, 4)                 # half the dilated span
    assert _args.resolve_padding("same", (2, 3), (1, 1), (1, 1)) == "same"                 # uneven: left to the local layer
    assert _args.resolve_padding(2, (3, 3), (2, 2), (1, 1)) == (2, 2)
    with pytest.raises(ValueError, match="strided"):
        _args.resolve_padding("same", (3, 3), (2, 1), (1, 1))
    with pytest.raises(ValueError, match="Invalid padding string"):
        _args.resolve_padding("full", (3, 3), (1, 1), (1, 1))


def test_channel_transport_names():
    assert _args.resolve_channel_comm("auto", "cpu") == "batch_isend_irecv"
    assert _args.resolve_channel_comm("auto", "cuda") == "all_to_all"
    assert _args.resolve_channel_comm("all_gather", "cpu") == "all_gather"
    for name in ("isend", "batch_isend_irecv", "ISEND"):
        assert _args.resolve_channel_comm(name, "cpu") == name.lower()
    from jigsaw_b200.modules import CommOp

    assert _args.resolve_channel_comm(CommOp.ISEND, "cpu") == "isend"
    with pytest.raises(ValueError, match="needs CUDA"):
        _args.resolve_channel_comm("all_to_all", "cpu")
    for bad in ("ring", "", "allgather"):
        with pytest.raises(ValueError, match="channel_comm must be"):
            _args.resolve_channel_comm(bad, "cpu")


def test_grouped_channels_against_the_channel_group():
    assert _args.resolve_conv_groups(1, 8, 16, 4) == (False, 1)                            # dense: channels travel
    assert _args.resolve_conv_groups(4, 8, 16, 4) == (True, 1) and _args.resolve_conv_groups(8, 8, 16, 4) == (True, 2)
    assert _args.resolve_conv_groups(1, 8, 16, 1) == (True, 1)
    with pytest.raises(ValueError, match="groups must be >= 1"):
        _args.resolve_conv_groups(0, 8, 16, 2)
    with pytest.raises(ValueError, match="divisible by groups"):
        _args.resolve_conv_groups(3, 8, 16, 1)
    with pytest.raises(ValueError, match="channel group size"):
        _args.resolve_conv_groups(1, 6, 16, 4)
    with pytest.raises(NotImplementedError, match="multiple of the channel-parallel group size"):
        _args.resolve_conv_groups(2, 8, 16, 4)


GEOMETRIES = [(3, 1, 1, 1), (5, 1, 2, 1), (3, 1, 2, 2), (4, 2, 1, 1), (2, 2, 0, 1), (3, 1, 0, 1), (7, 1, 3, 1)]


def _worker_halo(rank, world):
    import torch.distributed as dist
    import torch.nn.functional as F
    from jigsaw_b200.modules import CommOp
    from jigsaw_b200.modules.convolution import _halo

    group, comm = dist.group.WORLD, CommOp.BATCH_ISEND_IRECV
    n_local = 8
    gen = torch.Generator().manual_seed(1)
    x_full = torch.randn(2, 3, world * n_local, generator=gen, dtype=torch.float64)
    w = torch.randn(4, 3, 7, generator=gen, dtype=torch.float64)
    checked = 0
    for kernel, stride, padding, dilation in GEOMETRIES:
        tag = f"k={kernel} s={stride} p={padding} d={dilation}"
        try:
            plan, out_local = _halo.conv_axis_plan(-1, group, n_local, kernel, stride, padding, dilation, comm)
        except ValueError:                                      # this geometry's output does not divide over the ranks
            continue
        checked += 1
        x = split(x_full, {2: group})
        span = _halo.span_gather(x, plan)
        assert span.shape[-1] == plan.held
        got = F.conv1d(span, w[:, :, :kernel], stride=stride, dilation=dilation)            # no padding left to do
        want = F.conv1d(x_full, w[:, :, :kernel], stride=stride, padding=padding, dilation=dilation)
        assert_close(got, split(want, {2: group}), f"gather then local convolution, {tag}", 1e-12, 1e-12)
        # adjoint pair: sum over ranks of <gather(x), y> equals sum over ranks of <x, reduce(y)>
        y = torch.randn(span.shape, generator=torch.Generator().manual_seed(7 + rank), dtype=torch.float64)
        both = torch.stack(((span * y).sum(), (x * _halo.span_reduce(y, plan)).sum()))
        dist.all_reduce(both)
        assert all_ok(abs(float(both[0] - both[1])) < 1e-9 * max(1.0, abs(float(both[0])))), (tag, both)
        # and autograd uses exactly that
        leaf = x.clone().requires_grad_(True)
        (g,) = torch.autograd.grad(_halo.span_gather(leaf, plan), leaf, y)
        assert_close(g, _halo.span_reduce(y, plan), f"backward of gather is reduce, {tag}", 1e-12, 1e-12)
    assert checked >= 5, checked
    wt = torch.randn(3, 4, 7, generator=gen, dtype=torch.float64)
    for kernel, stride, padding, dilation in ((4, 2, 1, 1), (3, 1, 1, 1), (2, 2, 0, 1), (3, 2, 0, 1), (5, 1, 2, 1)):
        tag = f"transposed k={kernel} s={stride} p={padding}"
        try:
            plan = _halo.conv_transpose_axis_plan(-1, group, n_local, kernel, stride, padding, dilation, comm)
        except ValueError:
            continue
        x = split(x_full, {2: group})
        raw = F.conv_transpose1d(x, wt[:, :, :kernel], stride=stride, dilation=dilation)    # overhangs the tile
        assert raw.shape[-1] == plan.held
        got = _halo.span_reduce(raw, plan)
        want = F.conv_transpose1d(x_full, wt[:, :, :kernel], stride=stride, padding=padding, dilation=dilation)
        assert_close(got, split(want, {2: group}), f"local layer then reduce, {tag}", 1e-12, 1e-12)
        z = torch.randn(got.shape, generator=torch.Generator().manual_seed(9 + rank), dtype=torch.float64)
        both = torch.stack(((got * z).sum(), (raw * _halo.span_gather(z, plan)).sum()))
        dist.all_reduce(both)
        assert all_ok(abs(float(both[0] - both[1])) < 1e-9 * max(1.0, abs(float(both[0])))), (tag, both)
    # a plan whose output cannot be cut evenly is refused when it is made
    with pytest.raises(ValueError, match="divisible by the spatial group size"):
        _halo.conv_axis_plan(-1, group, n_local, 2, 1, 0, 1, comm)                           # an odd number of outputs


@pytest.mark.parametrize("world", [2, 4])
def test_halo_gather_and_reduce_are_an_adjoint_pair(world):
    run_distributed(_worker_halo, world, timeout=300)


def _worker_inputs(rank, world):
    import jigsaw_b200 as jb
    from jigsaw_b200.modules.convolution import ConvNdConfig, ConvTransposeNdConfig

    mesh = jb.make_process_mesh({"row": 2, "col": 2})
    M, row, col = jb.modules, mesh["row"], mesh["col"]
    for transposed in (False, True):
        cls = M.DistributedConvTranspose2d if transposed else M.DistributedConv2d
        layer = cls(4, 4, 3, "cpu", row, col, padding=1)
        for bad in (torch.randn(2, 6), torch.randn(1, 2, 2, 6, 3, 3)):
            with pytest.raises((ValueError, RuntimeError)):
                layer(bad)
        assert tuple(layer(torch.randn(2, 6, 3)).shape) == (2, 6, 3)                        # an image without a batch axis
        config_cls = ConvTransposeNdConfig if transposed else ConvNdConfig
        fits = config_cls(col, True, (3, 3), (1, 1), "cpu")
        cls(4, 4, 3, "cpu", row, col, padding=1, config=fits)
        for other in (config_cls(col, None, (3, 3), (1, 1), "cpu"), config_cls(col, True, (2, 2), (2, 2), "cpu"),
                      config_cls(col, True, (3,), (1,), "cpu"), config_cls(row, True, (3, 3), (1, 1), "cpu", groups=2)):
            with pytest.raises(ValueError, match="different layer"):
                cls(4, 4, 3, "cpu", row, col, padding=1, config=other)
    assert all_ok(True)


def test_inputs_of_the_wrong_rank_and_configurations_of_another_layer():
    run_distributed(_worker_inputs, 4, timeout=300)


def test_uneven_split_is_both_kinds_of_error():
    """An output that does not divide over the ranks is 'not supported' (the reference's type) and a wrong size."""
    from jigsaw_b200.modules import CommOp
    from jigsaw_b200.modules.convolution import _halo

    class Four:
        def size(self):
            return 4

    for make in (lambda: _halo.conv_axis_plan(-1, Four(), 8, 2, 1, 0, 1, CommOp.ISEND),
                 lambda: _halo.conv_transpose_axis_plan(-1, Four(), 8, 3, 2, 0, 1, CommOp.ISEND)):
        for kind in (NotImplementedError, ValueError, _halo.UnevenSplitError):
            with pytest.raises(kind, match="divisible by the spatial group size"):
                make()
