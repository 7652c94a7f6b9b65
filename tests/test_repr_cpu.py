"""``extra_repr`` of the distributed layers: the fields of the ``torch.nn`` (or serial) counterpart in the same
format, followed by the sizes of the process groups the layer is sharded over; re-sharding updates them.

Reference behaviours covered: tests/modules/test_repr.py:58-225.
"""

import pytest
import torch

from dist_utils import all_ok, run_distributed


def _with_bias(torch_repr, bias):
    """The ``bias`` field that older torch versions leave out of the norm reprs."""
    return torch_repr if "bias=" in torch_repr else f"{torch_repr}, bias={bias}"


def _worker_repr(rank, world, R, C):
    import jigsaw_b200 as jb
    from jigsaw_b200.modules import (Attention, DistributedAttention, DistributedConv2d, DistributedConvTranspose2d,
                                     DistributedCrossEntropyLoss, DistributedGroupNorm, DistributedL1Loss, DistributedLayerNorm,
                                     DistributedLinear, DistributedMatMulXWT, DistributedMSELoss, DistributedNLLLoss, DistributedRoll,
                                     DistributedSegmentationMetrics, DistributedSoftmax, Roll)

    mesh = jb.make_process_mesh({"row": R, "col": C})
    row, col, model = mesh["row"], mesh["col"], mesh["model"]

    def check(module, expected):
        got = module.extra_repr()
        assert all_ok(got == expected), f"{type(module).__name__}: {got!r} != {expected!r}"

    check(DistributedLinear(16, 32, "cpu", model, row, col, bias=False), f"{torch.nn.Linear(16, 32, bias=False).extra_repr()}, row={R}, col={C}")
    # with model_group == col_group the weight is replicated over the rows
    check(DistributedLinear(16, 32, "cpu", col, row, col), f"{torch.nn.Linear(16, 32).extra_repr()}, row=1, col={C}")
    check(DistributedMatMulXWT("cpu", model), f"model={R * C}")
    check(DistributedConv2d(4, 8, 3, "cpu", row, col, padding=(1,), bias=False),
          f"{torch.nn.Conv2d(4, 8, 3, padding=1, bias=False).extra_repr()}, spatial=(1, {R}), channel={C}")
    check(DistributedConvTranspose2d(4, 8, 2, "cpu", [row, None], col, stride=2),
          f"{torch.nn.ConvTranspose2d(4, 8, 2, stride=2).extra_repr()}, spatial=({R}, 1), channel={C}")
    check(DistributedLayerNorm(16, model.rank(), "cpu", row, col, eps=1e-6),
          f"{_with_bias(torch.nn.LayerNorm(16, eps=1e-6).extra_repr(), True)}, row={R}, col={C}")
    check(DistributedGroupNorm(4, 16, "cpu", channel_group=col, spatial_group=[row, row], affine=False),
          f"{_with_bias(torch.nn.GroupNorm(4, 16, affine=False).extra_repr(), False)}, spatial={R * R}, channel={C}")
    check(DistributedSoftmax(col, dim=1), f"{torch.nn.Softmax(dim=1).extra_repr()}, group={C}")
    check(DistributedRoll((1, 2), (1, 2), (2,), (col,), "cpu"), f"{Roll((1, 2), (1, 2)).extra_repr()}, distributed_dims=(2,), spatial=({C},)")
    check(DistributedAttention(16, 16, 8, 4, model.rank(), "cpu", row, col, qk_norm=True),
          f"{Attention(16, 16, 8, 4, 'cpu', qk_norm=True).extra_repr()}, ring=False, spatial={R}, channel={C}")
    check(DistributedL1Loss(), "reduce_groups=1")
    check(DistributedNLLLoss(), "channel=1, reduce_groups=1")
    check(DistributedMSELoss((row, col)), f"reduce_groups=({R}, {C})")
    check(DistributedCrossEntropyLoss(col, row), f"channel={C}, reduce_groups={R}")
    check(DistributedSegmentationMetrics(3, col, [row, None]), f"channel={C}, reduce_groups=({R}, 1)")
    if (R, C) == (2, 2):
        to_mesh = jb.make_process_mesh({"row": 1, "col": 4})
        layer = DistributedLinear(16, 32, "cpu", model, row, col)
        layer.reshard_parameters(mesh, to_mesh)
        check(layer, f"{torch.nn.Linear(16, 32).extra_repr()}, row=1, col=4")


@pytest.mark.parametrize("grid", [(1, 1), (2, 2), (1, 4), (4, 2)])
def test_extra_repr(grid):
    R, C = grid
    run_distributed(_worker_repr, R * C, R, C, timeout=300)
