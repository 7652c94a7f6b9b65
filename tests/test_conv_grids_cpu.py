"""Convolutions over tile grids of every shape: 3x2, 5x2, 1x4, 4x1, 2x1 (+ channel split), grouped and
transposed layers on two spatial axes, frozen parameters.

Every (grid, kernel, stride, padding, dilation) pair is either matched against the undivided torch layer in
float64 (output, input gradient, weight and bias gradient) or, when a split axis's global output does not
divide by that axis's ranks, refused with ``NotImplementedError`` / ``ValueError`` on every rank alike:
never silently wrong.

Reference behaviours covered: tests/modules/convolution/conv/test_conv2d_multi_spatial.py:441-660 (grid
sweep over 3x2, 1x4, 4x1, 2x2, 5x2, 2x1 and 2x1 with a channel split), :662-720 (grouped convolutions on a
two-axis split), tests/modules/convolution/conv_transpose/test_conv2dtranspose_multi_spatial.py (transposed
layers on a two-axis split), tests/modules/convolution/test_conv_grad_skip.py (frozen operands).
"""

import pytest
import torch

from dist_utils import all_ok, assert_close, run_distributed, split
from test_conv_cpu import _conv_case

# (kernel, stride, padding, dilation); ints or (h, w) pairs: no halo, stride < / > kernel, unit stride, dilated,
# asymmetric, stride == kernel pushed onto the halo path by padding or dilation
SWEEP = [
    (2, 2, 0, 1),
    (3, 2, 1, 1),
    (2, 3, 1, 1),
    (3, 1, 1, 1),
    (3, 1, 2, 2),
    ((3, 4), (2, 2), (1, 1), 1),
    ((4, 2), (2, 3), (1, 0), 1),
    (2, 2, 1, 1),
    ((3, 3), (3, 3), (0, 0), (1, 2)),
    (3, 2, 0, 1),
    (5, 1, 2, 1),
    ((1, 3), 1, (0, 1), 1),
]


def _worker_grid(rank, world, nh, nw, ncol, cases):
    import jigsaw_b200 as jb

    mesh = jb.make_process_mesh({"sh": nh, "sw": nw, "col": ncol})
    mesh["sd"] = None
    size = (12 * nh, 12 * nw)                                        # divides by the grid and by strides 2 and 3
    matched = refused = 0
    for i, (k, s, p, d) in enumerate(cases):
        try:
            _conv_case(mesh, 2, 2 * ncol, 4 * ncol, k, s, p, d, 1, False, "auto", size, 100 + i)
            matched += 1
        except (NotImplementedError, ValueError):
            refused += 1
    # the outcome is the same on every rank, and most of the sweep is computable
    assert all_ok(True)
    assert matched >= len(cases) // 2, (matched, refused)


@pytest.mark.parametrize("grid", [(3, 2, 1), (1, 4, 1), (4, 1, 1), (2, 1, 2), (2, 1, 1)],
                         ids=["3x2", "1x4", "4x1", "2x1_x2c", "2x1"])
def test_grid_sweep(grid):
    nh, nw, ncol = grid
    run_distributed(_worker_grid, nh * nw * ncol, nh, nw, ncol, SWEEP, timeout=600)


def test_grid_5x2():
    run_distributed(_worker_grid, 10, 5, 2, 1, SWEEP[:6], timeout=900)


def _worker_grouped_and_transposed(rank, world):
    import jigsaw_b200 as jb

    mesh = jb.make_process_mesh({"sh": 2, "sw": 2, "col": 1})
    mesh["sd"] = None
    for groups in (1, 2, 4, 8):                                       # no halo, then halo
        _conv_case(mesh, 2, 8, 16, 2, 2, 0, 1, groups, False, "auto", (8, 8), 200 + groups)
    for groups in (2, 4):
        _conv_case(mesh, 2, 8, 8, 3, 1, 1, 1, groups, False, "auto", (8, 12), 210 + groups)
    # transposed layers on two split axes: kernel == stride (no overlap), overlap with and without padding, asymmetric
    for i, (k, s, p) in enumerate([(2, 2, 0), (4, 2, 1), (3, 1, 1), ((4, 2), (2, 2), (1, 0)), ((3, 4), (1, 2), (1, 1)), (3, 3, 0)]):
        _conv_case(mesh, 2, 4, 6, k, s, p, 1, 1, True, "auto", (8, 12), 220 + i)
    for groups in (2, 4):
        _conv_case(mesh, 2, 8, 8, 4, 2, 1, 1, groups, True, "auto", (6, 8), 230 + groups)


def test_grouped_and_transposed_on_two_axes():
    run_distributed(_worker_grouped_and_transposed, 4, timeout=600)


def _worker_transposed_3d(rank, world):
    import jigsaw_b200 as jb

    mesh = jb.make_process_mesh({"sd": 2, "sh": 2, "sw": 2, "col": 1})
    for i, (k, s, p) in enumerate([(2, 2, 0), (4, 2, 1), (3, 1, 1), ((2, 4, 2), (2, 2, 2), (0, 1, 0))]):
        _conv_case(mesh, 3, 2, 4, k, s, p, 1, 1, True, "auto", (4, 6, 4), 300 + i)
    mesh2 = {"sd": None, "sh": mesh["sh"], "sw": mesh["sw"], "col": mesh["sd"]}      # the same ranks as 2 x 2 tiles + 2 channel ranks
    for i, (k, s, p) in enumerate([(3, 1, 1), (2, 2, 0), (3, 2, 1)]):
        _conv_case(mesh2, 2, 4, 8, k, s, p, 1, 1, False, "auto", (8, 8), 310 + i)
        if k >= s:
            _conv_case(mesh2, 2, 4, 8, k + (k - s) % 2, s, p, 1, 1, True, "auto", (8, 8), 320 + i)


def test_transposed_3d_and_channel_split_on_eight_ranks():
    run_distributed(_worker_transposed_3d, 8, timeout=900)


def _worker_frozen(rank, world):
    """Frozen operands: a layer whose weight (or whose input) needs no gradient skips that gradient's
    collectives on every rank alike, returns ``None`` for it and still gives the others exactly."""
    import jigsaw_b200 as jb

    mesh = jb.make_process_mesh({"sh": 2, "sw": 1, "col": 2})
    sh, col = mesh["sh"], mesh["col"]
    M = jb.modules
    torch.manual_seed(5)
    for transposed in (False, True):
        cls, tcls = (M.DistributedConvTranspose2d, torch.nn.ConvTranspose2d) if transposed else (M.DistributedConv2d, torch.nn.Conv2d)
        k, s, p = (4, 2, 1) if transposed else (3, 1, 1)
        ref = tcls(4, 8, k, stride=s, padding=p).double()
        x = torch.randn(2, 4, 8, 6, dtype=torch.float64)
        cuts = {1: col, 2: sh}
        for frozen in ("weight", "bias", "input", "all_parameters"):
            ref.zero_grad()
            ref.weight.requires_grad_(frozen not in ("weight", "all_parameters"))
            ref.bias.requires_grad_(frozen not in ("bias", "all_parameters"))
            xr = x.clone().requires_grad_(frozen != "input")
            yr = ref(xr)
            g = torch.randn_like(yr)
            if yr.requires_grad:
                yr.backward(g)
            layer = cls(4, 8, k, "cpu", (sh, None), col, stride=s, padding=p, dtype=torch.float64)
            layer._load_global(ref.weight.data, ref.bias.data)
            layer.weight.requires_grad_(ref.weight.requires_grad)
            layer.bias.requires_grad_(ref.bias.requires_grad)
            xl = split(x, cuts).requires_grad_(frozen != "input")
            y = layer(xl)
            tag = f"T={transposed} frozen={frozen}"
            assert_close(y, split(yr.detach(), cuts), f"{tag}: output", 1e-10, 1e-10)
            y.backward(split(g, cuts))
            wdim = layer._weight_shard_dim
            for name, mine, full, cut in (("dx", xl.grad, xr.grad, cuts), ("dW", layer.weight.grad, ref.weight.grad, {wdim: col}),
                                         ("db", layer.bias.grad, ref.bias.grad, {0: col})):
                if full is None:
                    assert mine is None, f"{tag}: {name} must stay None"
                else:
                    assert_close(mine, split(full, cut), f"{tag}: {name}", 1e-10, 1e-10)


def test_frozen_operands_skip_their_collectives():
    run_distributed(_worker_frozen, 4, timeout=600)


STRING_PADDINGS = {"valid_patchify": (2, 2, "valid", 1), "same_k1": (1, 1, "same", 1), "same_k3": (3, 1, "same", 1),
                   "same_k3_dilated": (3, 1, "same", 2), "same_k5": (5, 1, "same", 1)}
CHANNEL_COMMS = ("all_gather", "isend", "batch_isend_irecv")


def _worker_string_padding(rank, world, axes, name):
    """``padding="valid"`` / ``"same"`` on a layer cut in space and channels, with every way of moving channels,
    against the undivided layer given the same string (reference: tests/modules/convolution/conv/
    test_convolution_2d.py:755-824)."""
    import jigsaw_b200 as jb

    mesh = jb.make_process_mesh(axes)
    mesh["sd"] = mesh["sh"] = None
    mesh["sw"] = mesh["row"]
    k, s, p, d = STRING_PADDINGS[name]
    C = mesh["col"].size()
    for channel_comm in CHANNEL_COMMS:
        _conv_case(mesh, 2, 2 * C, 4 * C, k, s, p, d, 1, False, channel_comm, (6, 12 * mesh["row"].size()), 7)
    _conv_case(mesh, 1, 2 * C, 4 * C, k, s, p, d, 1, False, "auto", (12 * mesh["row"].size(),), 8)


@pytest.mark.parametrize("name", list(STRING_PADDINGS))
def test_string_padding_on_2x2(name):
    run_distributed(_worker_string_padding, 4, {"row": 2, "col": 2}, name, timeout=300)


def _worker_rectangular(rank, world, axes):
    """Meshes that are not powers of two: 2-way space x 3-way channels and the other way round, every way of moving
    channels, plain and transposed (reference: test_convolution_2d.py:901-935)."""
    import jigsaw_b200 as jb

    mesh = jb.make_process_mesh(axes)
    mesh["sd"] = mesh["sh"] = None
    mesh["sw"] = mesh["row"]
    R, C = mesh["row"].size(), mesh["col"].size()
    for channel_comm in CHANNEL_COMMS:
        _conv_case(mesh, 2, 2 * C, 3 * C, 3, 1, 1, 1, 1, False, channel_comm, (5, 4 * R), 11)
        _conv_case(mesh, 2, 2 * C, 3 * C, 2, 2, 0, 1, 1, False, channel_comm, (4, 4 * R), 12)
        _conv_case(mesh, 2, 2 * C, 3 * C, 4, 2, 1, 1, 1, True, channel_comm, (3, 2 * R), 13)
    _conv_case(mesh, 2, 2 * C, 4 * C, 3, 1, 1, 1, C, False, "auto", (5, 4 * R), 14)                   # whole groups per rank


@pytest.mark.parametrize("axes", [{"row": 2, "col": 3}, {"row": 3, "col": 2}], ids=["2x3", "3x2"])
def test_rectangular_meshes_with_channel_split(axes):
    run_distributed(_worker_rectangular, 6, axes, timeout=400)


TRANSPOSED_CASES = [(2, 2, 0), (4, 2, 1), (3, 1, 1), (3, 2, 0), (5, 1, 2), (4, 4, 0)]          # (kernel, stride, padding)


def _worker_transposed_meshes(rank, world, axes):
    """Transposed layers on channel-only, space-only and mixed meshes, every way of moving channels, with and
    without an overhang to hand to the neighbours (reference: conv_transpose/test_conv2dtranspose.py:350-590)."""
    import jigsaw_b200 as jb

    mesh = jb.make_process_mesh(axes)
    mesh["sd"] = mesh["sh"] = None
    mesh["sw"] = mesh["row"]
    R, C = mesh["row"].size(), mesh["col"].size()
    matched = 0
    for channel_comm in CHANNEL_COMMS:
        for i, (k, s, p) in enumerate(TRANSPOSED_CASES):
            try:
                _conv_case(mesh, 2, 2 * C, 2 * C, k, s, p, 1, 1, True, channel_comm, (3, 4 * R), 30 + i)
                matched += 1
            except (NotImplementedError, ValueError):
                pass                                          # an output that does not divide over the ranks: refused alike
    assert all_ok(True) and matched >= 3 * 4, matched
    with pytest.raises(NotImplementedError, match="string padding"):
        jb.modules.DistributedConvTranspose2d(2 * C, 2 * C, 3, "cpu", mesh["row"], mesh["col"], padding="same")
    if C > 1:                                                 # groups that do not stay whole on a channel rank
        with pytest.raises(NotImplementedError, match="multiple of the channel-parallel group size"):
            jb.modules.DistributedConvTranspose2d(6 * C, 6 * C, 3, "cpu", mesh["row"], mesh["col"], groups=3)


@pytest.mark.parametrize("axes", [{"row": 1, "col": 4}, {"row": 4, "col": 1}, {"row": 2, "col": 2}, {"row": 2, "col": 4}],
                         ids=["1x4", "4x1", "2x2", "2x4"])
def test_transposed_layers_on_channel_space_and_mixed_meshes(axes):
    run_distributed(_worker_transposed_meshes, axes["row"] * axes["col"], axes, timeout=600)
