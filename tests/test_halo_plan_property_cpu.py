"""Span arithmetic of the halo plans against brute force, on drawn geometries (no processes: a plan only asks its
group for a size).

For a convolution axis cut over G ranks, rank q computes outputs [q * out_local, (q + 1) * out_local); output o
reads inputs o * stride - padding + j * dilation for j < kernel.  The plan's held span must be exactly the hull of
those reads.  For a transposed axis, rank q's raw local output covers the positions i * stride + j * dilation -
padding of its inputs i; the plan's held span must be that hull, the owned ranges must tile the global output,
and every produced position inside the domain must fall into some rank's owned range.
"""

import pytest

hypothesis = pytest.importorskip("hypothesis")
from hypothesis import given, settings  # noqa: E402
from hypothesis import strategies as st  # noqa: E402

from jigsaw_b200.modules import CommOp  # noqa: E402
from jigsaw_b200.modules.convolution import _halo  # noqa: E402


class _Group:
    def __init__(self, size):
        self._size = size

    def size(self):
        return self._size

    def rank(self):
        return 0


geometry = st.tuples(st.integers(1, 6), st.integers(1, 24), st.integers(1, 7), st.integers(1, 4), st.integers(0, 6), st.integers(1, 3))


@settings(max_examples=400, deadline=None)
@given(geometry)
def test_convolution_plan_holds_exactly_what_its_outputs_read(g):
    G, n_local, kernel, stride, padding, dilation = g
    extent = dilation * (kernel - 1) + 1
    total_out = (G * n_local + 2 * padding - extent) // stride + 1
    try:
        plan, out_local = _halo.conv_axis_plan(-1, _Group(G), n_local, kernel, stride, padding, dilation, CommOp.ISEND)
    except ValueError:
        assert total_out <= 0 or total_out % G != 0
        return
    assert total_out > 0 and total_out % G == 0 and out_local * G == total_out
    assert plan.own == n_local and plan.total == G * n_local and len(plan.lo) == G
    for q in range(G):
        reads = [o * stride - padding + j * dilation for o in range(q * out_local, (q + 1) * out_local) for j in range(kernel)]
        assert plan.lo[q] == min(reads) and plan.lo[q] + plan.held == max(reads) + 1
        for owner in range(G):                                     # what q holds of owner's tile: inside both, inside the domain
            a, b = plan.overlap(q, owner)
            assert a <= b
            if a < b:
                assert owner * n_local <= a and b <= (owner + 1) * n_local and plan.lo[q] <= a and b <= plan.lo[q] + plan.held
        covered = sum(b - a for a, b in (plan.overlap(q, owner) for owner in range(G)))
        inside = len([p for p in range(plan.lo[q], plan.lo[q] + plan.held) if 0 <= p < plan.total])
        assert covered == inside                                   # every in-domain position of the span has exactly one owner


@settings(max_examples=400, deadline=None)
@given(geometry)
def test_transposed_plan_covers_what_its_inputs_produce(g):
    G, n_local, kernel, stride, padding, dilation = g
    extent = dilation * (kernel - 1) + 1
    total_out = (G * n_local - 1) * stride - 2 * padding + extent
    try:
        plan = _halo.conv_transpose_axis_plan(-1, _Group(G), n_local, kernel, stride, padding, dilation, CommOp.ISEND)
    except ValueError:
        assert total_out <= 0 or total_out % G != 0
        return
    assert total_out > 0 and plan.total == total_out and plan.own * G == total_out
    for q in range(G):
        writes = [i * stride + j * dilation - padding for i in range(q * n_local, (q + 1) * n_local) for j in range(kernel)]
        assert plan.lo[q] == min(writes) and plan.lo[q] + plan.held == max(writes) + 1
        for p in set(writes):
            if 0 <= p < total_out:
                owner = p // plan.own
                a, b = plan.overlap(q, owner)
                assert a <= p < b                                  # the owner of p receives it from q
