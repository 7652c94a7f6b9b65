"""Two ways of counting the parameters of the whole model, both against the torch layer's ``numel``.

``get_parameter_count`` is computed by each layer from its global shapes, without communication, and must be the
whole layer's count on every rank.  ``debug.count_parameters(module, mesh)`` adds up the pieces that the ranks
really hold and counts a replicated parameter once per replica group, so it only meets the torch count when
every replicated parameter carries its mark and no sharded one does: a missing mark counts the parameter once
per rank (and its gradient would never be summed), a mark too many loses pieces.

Reference behaviours covered: tests/test_param_count.py (layer table on 2 x 2, group norm on channels only, both
counts).
"""

import pytest
import torch

from dist_utils import all_ok, run_distributed


class _AttentionParameters(torch.nn.Module):
    """The parameters an undivided attention layer of this width has."""

    def __init__(self, dim, heads, qk_norm, bias=True):
        super().__init__()
        self.qkv = torch.nn.Linear(dim, 3 * dim, bias=False)
        self.out = torch.nn.Linear(dim, dim, bias=bias)
        if qk_norm:
            self.q_norm, self.k_norm = torch.nn.LayerNorm(dim // heads), torch.nn.LayerNorm(dim // heads)


def _table(mesh):
    import jigsaw_b200 as jb

    M, nn = jb.modules, torch.nn
    row, col, model = mesh["row"], mesh["col"], mesh["model"]
    conv_kw = dict(device="cpu", spatial_group=row, channel_group=col)

    def linear(i, o, bias=True):
        return M.DistributedLinear(i, o, "cpu", model, row, col, bias=bias)

    def attention(qk_norm, ring=False, bias=True):
        return M.DistributedAttention(8, 8, 8, 4, col.rank(), "cpu", row, col, qk_norm=qk_norm, ring=ring, out_bias=bias,
                                      attn_backend="math")

    rows = [
        ("layer norm", lambda: M.DistributedLayerNorm(8, model.rank(), "cpu", row, col), nn.LayerNorm(8)),
        ("group norm", lambda: M.DistributedGroupNorm(4, 8, "cpu", channel_group=col, spatial_group=row), nn.GroupNorm(4, 8)),
        ("linear", lambda: linear(8, 16), nn.Linear(8, 16)),
        ("linear, no bias", lambda: linear(8, 16, False), nn.Linear(8, 16, bias=False)),
        ("mlp", lambda: nn.Sequential(linear(8, 16), nn.GELU(), linear(16, 8)),
         nn.Sequential(nn.Linear(8, 16), nn.GELU(), nn.Linear(16, 8))),
        ("attention", lambda: attention(False), _AttentionParameters(8, 4, False)),
        ("attention, qk norm", lambda: attention(True), _AttentionParameters(8, 4, True)),
        ("attention, no output bias", lambda: attention(False, bias=False), _AttentionParameters(8, 4, False, bias=False)),
    ]
    if row.size() == 1:                       # without a spatial group the layer cannot know of copies over the rows
        rows.append(("group norm, channels only", lambda: M.DistributedGroupNorm(4, 8, "cpu", channel_group=col), nn.GroupNorm(4, 8)))
    if row.size() > 1:
        rows.append(("attention, ring", lambda: attention(True, ring=True), _AttentionParameters(8, 4, True)))
    for groups in (1, 2, 4):
        for bias in (True, False):
            if (groups > 1 and not bias) or (groups > 1 and groups % col.size()):
                continue                          # grouped channels must stay whole on a rank
            rows.append((f"conv2d groups={groups} bias={bias}",
                         lambda g=groups, b=bias: M.DistributedConv2d(8, 16, 3, groups=g, bias=b, **conv_kw),
                         nn.Conv2d(8, 16, 3, groups=groups, bias=bias)))
    for bias in (True, False):
        rows.append((f"conv transpose 2d bias={bias}", lambda b=bias: M.DistributedConvTranspose2d(8, 16, 3, bias=b, **conv_kw),
                     nn.ConvTranspose2d(8, 16, 3, bias=bias)))
    rows.append(("conv1d", lambda: M.DistributedConv1d(8, 8, 5, **conv_kw), nn.Conv1d(8, 8, 5)))
    rows.append(("conv3d", lambda: M.DistributedConv3d(4, 8, 3, "cpu", (row, None, None), col), nn.Conv3d(4, 8, 3)))
    return rows


def _computed(module):
    """Sum of the layers' own reports.  A layer with ``get_parameter_count`` answers for its direct parameters and
    for children made of plain torch modules only (the q/k norms inside attention); children that can answer do
    so themselves; a container without the method adds its direct parameters."""
    answers = hasattr(module, "get_parameter_count")
    total = module.get_parameter_count() if answers else sum(p.numel() for p in module.parameters(recurse=False))
    for child in module.children():
        plain = not any(hasattr(m, "get_parameter_count") for m in child.modules())
        if not (answers and plain):
            total += _computed(child)
    return total


def _worker(rank, world, axes):
    import jigsaw_b200 as jb

    mesh = jb.make_process_mesh(axes)
    wrong = []
    for label, build, reference in _table(mesh):
        want = sum(p.numel() for p in reference.parameters())
        module = build()
        held = jb.debug.count_parameters(module, mesh)
        computed = _computed(module)
        if not all_ok(held == want):
            wrong.append(f"{label}: the ranks hold {held} parameters, torch has {want}")
        if not all_ok(computed == want):
            wrong.append(f"{label}: get_parameter_count gives {computed}, torch has {want}")
    assert not wrong, (axes, wrong)


@pytest.mark.parametrize("axes", [{"row": 2, "col": 2}, {"row": 1, "col": 4}, {"row": 4, "col": 1}], ids=["2x2", "1x4", "4x1"])
def test_counts_match_the_torch_layers(axes):
    run_distributed(_worker, 4, axes, timeout=600)


def _worker_marks(rank, world):
    """What the held count does with a mark that is missing or too many."""
    import jigsaw_b200 as jb
    from jigsaw_b200.parallel._replicas import MARK_ATTR

    mesh = jb.make_process_mesh({"row": 2, "col": 2})
    layer = jb.modules.DistributedLinear(8, 16, "cpu", mesh["model"], mesh["row"], mesh["col"])
    assert all_ok(jb.debug.count_parameters(layer, mesh) == 8 * 16 + 16)
    groups = jb.parallel.replica_groups(layer.bias)
    assert [g.size() for g in groups] == [2]                                    # the bias: alike over the row ranks
    delattr(layer.bias, MARK_ATTR)
    assert all_ok(jb.debug.count_parameters(layer, mesh) == 8 * 16 + 2 * 16)    # mark gone: counted once per row rank
    jb.parallel.mark_replicated(layer.bias, groups)
    jb.parallel.mark_replicated(layer.weight, (mesh["col"],))
    assert all_ok(jb.debug.count_parameters(layer, mesh) == 8 * 16 // 2 + 16)   # a mark too many: half the pieces lost


def test_held_count_shows_a_missing_or_spurious_mark():
    run_distributed(_worker_marks, 4, timeout=300)
