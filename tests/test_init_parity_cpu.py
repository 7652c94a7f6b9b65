"""Freshly built layers start from the distribution of their torch counterparts.

``torch.nn.Linear`` and the (transposed) convolutions draw weight and bias uniformly within 1 / sqrt(fan_in) of
the whole layer.  A rank only fills its piece, so the bound must come from the whole layer's fan; were it taken
from the piece, the gathered parameter would still be uniform, only over the wrong range, and no comparison of
sharded against undivided outputs with copied weights would notice.  So: build, gather, and check that the
largest magnitude is within the bound and (thousands of draws) above 85 % of it.

Reference behaviours covered: tests/modules/test_init_parity.py (linear, convolutions and transposed convolutions
in one to three dimensions, overriding ``reset_parameters``).
"""

import math

import pytest

from dist_utils import all_ok, run_distributed


def _within(t, bound):
    top = float(t.abs().max())
    return 0.85 * bound < top <= bound + 1e-6


def _worker(rank, world, axes):
    import jigsaw_b200 as jb

    mesh = jb.make_process_mesh(axes)
    M, row, col = jb.modules, mesh["row"], mesh["col"]
    jb.launch.set_all_seeds(1 + rank)                     # independent draws on every rank
    wrong = []
    lin = M.DistributedLinear(64, 128, "cpu", mesh["model"], row, col)
    w, b = lin.merge_weights(mesh)
    if not all_ok(tuple(w.shape) == (128, 64) and tuple(b.shape) == (128,) and _within(w, 1 / 8) and _within(b, 1 / 8)):
        wrong.append(f"linear: max |w| {float(w.abs().max()):.4f}, max |b| {float(b.abs().max()):.4f}, bound {1 / 8:.4f}")
    cin, cout, k = 8, 32, 3
    for n in (1, 2, 3):
        spatial = (row,) + (None,) * (n - 1)
        for transposed in (False, True):
            cls = getattr(M, f"DistributedConv{'Transpose' if transposed else ''}{n}d")
            conv = cls(cin, cout, k, "cpu", spatial, col)
            w, b = conv.merge_weights(mesh)
            shape = (cin, cout) if transposed else (cout, cin)
            fan_in = shape[1] * k ** n                     # torch reads the fan off axis 1 of the weight
            ok = tuple(w.shape) == (*shape, *([k] * n)) and tuple(b.shape) == (cout,)
            bound = 1 / math.sqrt(fan_in)
            ok = ok and _within(w, bound) and 0.5 * bound < float(b.abs().max()) <= bound + 1e-6      # the bias has only 32 draws
            if not all_ok(ok):
                wrong.append(f"{cls.__name__}: max |w| {float(w.abs().max()):.4f}, bound {1 / math.sqrt(fan_in):.4f}")
    assert not wrong, (axes, wrong)

    class Constant(M.DistributedConv2d):
        def reset_parameters(self):
            jb.init.zeros_(self.weight)
            if self.bias is not None:
                jb.init.constant_(self.bias, 0.5)

    conv = Constant(cin, cout, k, "cpu", (row, None), col)
    assert not conv.weight.any() and bool((conv.bias == 0.5).all())

    class Wide(M.DistributedLinear):
        def reset_parameters(self):
            jb.init.xavier_uniform_(self.weight, global_shape=self.global_weight_shape)
            jb.init.zeros_(self.bias)

    lin = Wide(64, 128, "cpu", mesh["model"], row, col)
    w, b = lin.merge_weights(mesh)
    assert all_ok(_within(w, math.sqrt(6 / (64 + 128)))) and not b.any()


@pytest.mark.parametrize("axes", [{"row": 2, "col": 2}, {"row": 1, "col": 4}], ids=["2x2", "1x4"])
def test_fresh_layers_use_the_bounds_of_the_whole_layer(axes):
    run_distributed(_worker, 4, axes, timeout=300)
