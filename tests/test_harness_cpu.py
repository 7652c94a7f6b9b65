"""The multi-process harness of this test suite (``dist_utils``): what a failing, dying or hanging rank does to
the test, and the helpers that cut, gather and compare tensors.  A harness that hid a failing rank would make
every other multi-rank test worthless, so it is tested like the library.

Counterpart of the reference's tests of its own harness (tests/test_mesh_fixture.py); the harness here spawns
its ranks and needs no MPI.
"""

import os
import time

import pytest
import torch

from dist_utils import all_ok, assert_close, merge, run_distributed, singleton_mesh, split


def _worker_fails_on_one_rank(rank, world):
    if rank == 1:
        raise ValueError("rank one does not like this")


def _worker_exits_without_a_word(rank, world):
    if rank == 1:
        os._exit(3)
    time.sleep(30)


def _worker_never_finishes(rank, world):
    if rank == 0:
        time.sleep(60)


def _worker_disagreement(rank, world):
    assert_close(torch.full((2,), float(rank == 2)), torch.zeros(2), "deliberately wrong on rank 2", 0, 0)


def test_an_exception_on_one_rank_fails_the_test_with_its_traceback():
    with pytest.raises(AssertionError, match=r"rank 1 failed:(.|\n)*ValueError: rank one does not like this"):
        run_distributed(_worker_fails_on_one_rank, 3, timeout=120)


def test_a_rank_that_dies_is_reported_at_once():
    start = time.monotonic()
    with pytest.raises(AssertionError, match=r"died without reporting.*\(1, 3\)"):
        run_distributed(_worker_exits_without_a_word, 2, timeout=120)
    assert time.monotonic() - start < 60, "the harness waited for the time limit although a rank was dead"


def test_a_rank_that_hangs_runs_into_the_time_limit():
    with pytest.raises(AssertionError, match="timeout: only ranks"):
        run_distributed(_worker_never_finishes, 2, timeout=8)


def test_a_mismatch_on_one_rank_raises_on_every_rank():
    with pytest.raises(AssertionError, match="deliberately wrong on rank 2: mismatch on some rank"):
        run_distributed(_worker_disagreement, 3, timeout=120)


def _worker_helpers(rank, world):
    import jigsaw_b200 as jb

    mesh = jb.make_process_mesh({"row": 2, "col": 2})
    full = torch.arange(2 * 4 * 6, dtype=torch.float32).view(2, 4, 6)
    cuts = {1: mesh["row"], 2: mesh["col"], 0: None}
    piece = split(full, cuts)
    r, c = mesh["row"].rank(), mesh["col"].rank()
    assert torch.equal(piece, full[:, 2 * r:2 * r + 2, 3 * c:3 * c + 3]) and piece.is_contiguous()
    piece += 1                                                   # a copy: the global tensor stays as it was
    assert float(full[0, 0, 0]) == 0.0
    assert torch.equal(merge(piece - 1, cuts), full)
    assert all_ok(True) and not all_ok(rank != 3) and all_ok(True)
    solo = singleton_mesh("row", "col")
    assert set(solo) == {"row", "col", "model"} and all(g.size() == 1 and g.rank() == 0 for g in solo.values())
    assert torch.equal(split(full, {1: solo["row"]}), full)
    assert os.environ["RANK"] == str(rank) and os.environ["WORLD_SIZE"] == "4" and torch.get_num_threads() == 1


def test_split_merge_agreement_and_single_rank_meshes():
    run_distributed(_worker_helpers, 4, timeout=120)
