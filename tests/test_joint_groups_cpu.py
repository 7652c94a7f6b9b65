"""The joint groups of the DDP communication hook as pure arithmetic: ranks joined by the data-parallel groups and
by every replica group of a parameter form connected components; each component is one reduction group.  Also the
cache of created groups, with group creation faked.

Reference behaviours covered: tests/test_parallel.py:283-352 (dp x row, uneven tuples, the fully connected case,
groups that join nothing, singletons, interleaved parts, a long chain, the cache).
"""

import torch.distributed as dist

from jigsaw_b200.parallel import _joint

# 2 x 2 x 2 mesh, rank = 4 * dp + 2 * row + col
DP = [[0, 4], [1, 5], [2, 6], [3, 7]]
ROW = [[0, 2], [1, 3], [4, 6], [5, 7]]
COL = [[0, 1], [2, 3], [4, 5], [6, 7]]


def test_components():
    comp = _joint._components
    assert comp(8, DP + ROW) == [[0, 2, 4, 6], [1, 3, 5, 7]]                 # the bias of a linear layer: dp x row
    assert comp(8, DP + COL) == [[0, 1, 4, 5], [2, 3, 6, 7]]                 # a weight replicated over col
    assert comp(8, DP + ROW + COL) == [list(range(8))]                       # dp x row x col is every rank
    assert comp(8, [[0, 2, 4, 6], [1, 3, 5, 7], [0, 1], [2, 3], [4, 5], [6, 7]]) == [list(range(8))]
    assert comp(8, DP) == DP                                                  # no replica group joins nothing
    assert comp(4, []) == [[0], [1], [2], [3]]
    assert comp(8, [[0, 2, 5], [1, 4], [3, 6, 7]]) == [[0, 2, 5], [1, 4], [3, 6, 7]]   # parts need not be contiguous; sorted by rank
    # 7-3-5-1-6-2-4-0: every list links only neighbours, the smallest label has to travel the whole chain
    assert comp(8, [[7, 3], [5, 1], [6, 2], [4, 0], [3, 5], [1, 6], [2, 4]]) == [list(range(8))]
    assert comp(3, [[2], [1]]) == [[0], [1], [2]]                             # one-rank lists join nothing


def test_groups_are_created_once_per_partition(monkeypatch):
    made = []

    def fake(partition):
        made.append(partition)
        return f"group {len(made)}", []

    monkeypatch.setattr(_joint, "_partition_cache", {})
    monkeypatch.setattr(dist, "new_subgroups_by_enumeration", fake)
    part = _joint._components(8, DP + ROW)
    a = _joint._group_for_partition(part)
    b = _joint._group_for_partition(_joint._components(8, [[0, 2, 4, 6], [1, 3, 5, 7]]))   # other lists, same partition
    assert a == b == "group 1" and made == [part]
    assert _joint._group_for_partition(DP) == "group 2" and made == [part, DP]
    assert _joint._group_for_partition([list(range(8))]) is dist.group.WORLD and len(made) == 2   # every rank: the world, no new group
