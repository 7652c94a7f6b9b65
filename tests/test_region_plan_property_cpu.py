"""The plan behind ``fetch_region`` against brute force, on drawn grids (no processes: the plan asks its group for
a rank only).

A matrix is cut into R x C blocks of h x w elements, block (i, j) on rank i * C + j.  Every rank names a region it
wants; the plan says which piece of which block to send where.  Checked: the pieces a rank receives tile its
region exactly (every wanted element from the one block that owns it, nothing twice); what rank q plans to send to
rank p is what rank p plans to receive from rank q; and regions used by the layers (a row of blocks, a column of
blocks, the transposed swap) come out as expected.
"""

import pytest

hypothesis = pytest.importorskip("hypothesis")
from hypothesis import given, settings  # noqa: E402
from hypothesis import strategies as st  # noqa: E402

from jigsaw_b200.modules.linear._functional import _plan  # noqa: E402


class _Rank:
    def __init__(self, rank):
        self._rank = rank

    def rank(self):
        return self._rank


grids = st.tuples(st.integers(1, 4), st.integers(1, 4), st.integers(1, 5), st.integers(1, 5))


def _regions(draw, R, C, h, w):
    out = []
    for _ in range(R * C):
        r0 = draw(st.integers(0, R * h - 1))
        c0 = draw(st.integers(0, C * w - 1))
        out.append((r0, draw(st.integers(r0 + 1, R * h)), c0, draw(st.integers(c0 + 1, C * w))))
    return out


@settings(max_examples=200, deadline=None)
@given(st.data())
def test_received_pieces_tile_the_wanted_region_and_match_the_senders(data):
    R, C, h, w = data.draw(grids)
    regions = _regions(data.draw, R, C, h, w)
    plans = [_plan(h, w, _Rank(p), R, C, lambda q: regions[q]) for p in range(R * C)]
    for me, (mine, want, send, recv) in enumerate(plans):
        assert mine == ((me // C) * h, (me // C + 1) * h, (me % C) * w, (me % C + 1) * w) and want == regions[me]
        seen = set()
        for p, (r0, r1, c0, c1) in recv.items():
            assert r0 < r1 and c0 < c1
            for r in range(r0, r1):
                for c in range(c0, c1):
                    assert (r // h) * C + c // w == p, "an element must come from the rank whose block holds it"
                    assert (r, c) not in seen
                    seen.add((r, c))
        assert seen == {(r, c) for r in range(want[0], want[1]) for c in range(want[2], want[3])}
        for p, piece in send.items():
            assert plans[p][3][me] == piece, "what I send to p is what p expects from me"
        assert set(send) == {p for p in range(R * C) if me in plans[p][3]}


@pytest.mark.parametrize("R, C", [(1, 1), (2, 2), (1, 4), (4, 2), (3, 2)])
def test_regions_the_layers_use(R, C):
    h, w = 3, 5
    for me in range(R * C):
        i, j = divmod(me, C)
        _, _, send, recv = _plan(h, w, _Rank(me), R, C, lambda p: ((p // C) * h, (p // C + 1) * h, 0, w * C))      # my row of blocks
        assert sorted(recv) == [i * C + c for c in range(C)] and sorted(send) == sorted(recv)
        _, _, send, recv = _plan(h, w, _Rank(me), R, C, lambda p: (0, h * R, (p % C) * w, (p % C + 1) * w))         # my column of blocks
        assert sorted(recv) == [r * C + j for r in range(R)] and sorted(send) == sorted(recv)
        _, want, _, recv = _plan(h, w, _Rank(me), R, C, lambda p: (0, h * R, 0, w * C))                              # everything
        assert sorted(recv) == list(range(R * C)) and want == (0, h * R, 0, w * C)
