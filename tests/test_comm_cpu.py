"""Communication primitives: transport resolution, the sparse exchange over every CPU transport (uneven tables,
idle peers, self entries, asynchronous completion), ring shifts in both directions, the scalar MAX-reduce, backend
checks.

Reference behaviours covered: tests/test_comm.py:121-150 (transport resolution), :182-250 (two-rank ring shifts,
strided views, explicit peers, broadcast), :251-260 (a ring on a fresh group).
"""

import pytest
import torch

from dist_utils import assert_close, run_distributed


def test_transport_resolution():
    from jigsaw_b200._core.comm import CommOp, resolve_comm_op

    assert resolve_comm_op("auto", "cpu") is CommOp.BATCH_ISEND_IRECV
    assert resolve_comm_op(CommOp.AUTO, "cuda") is CommOp.ALL_TO_ALL
    for value in ("isend", "ISEND", "Batch_Isend_Irecv", CommOp.ISEND, CommOp.BATCH_ISEND_IRECV):
        assert isinstance(resolve_comm_op(value, "cpu"), CommOp)
    assert resolve_comm_op("isend", "cuda") is CommOp.BATCH_ISEND_IRECV      # separate NCCL sends around a ring can deadlock
    assert str(CommOp.ALL_TO_ALL) == "all_to_all"
    with pytest.raises(ValueError, match="needs CUDA"):
        resolve_comm_op("all_to_all", "cpu")
    with pytest.raises(ValueError, match="comm must be one of"):
        resolve_comm_op("carrier_pigeon", "cpu")
    with pytest.raises(ValueError, match="Unsupported device"):
        resolve_comm_op("auto", "meta")


def _worker_exchange(rank, world):
    import jigsaw_b200 as jb
    import torch.distributed as dist
    from jigsaw_b200._core.comm import (CommOp, all_reduce_max, check_backend, get_device_of_process_group, ring_shift,
                                        sparse_exchange)

    g = dist.group.WORLD
    assert check_backend(g) == {"gloo"} and get_device_of_process_group(g) == torch.device("cpu")
    for comm in (CommOp.BATCH_ISEND_IRECV, CommOp.ISEND):
        # uneven table: rank r sends r + 1 + p values to p; rank 0 sends nothing to rank 1 (an idle pair)
        sends = {p: torch.full((rank + 1 + p,), float(10 * rank + p)) for p in range(world) if not (rank == 0 and p == 1)}
        recvs = {p: torch.empty(p + 1 + rank) for p in range(world) if not (p == 0 and rank == 1)}
        sparse_exchange(sends, recvs, g, comm)
        for p, buf in recvs.items():
            assert torch.all(buf == 10 * p + rank), (comm, rank, p, buf)
        # asynchronous form; a strided view must be made contiguous by the caller, a 2-D payload keeps its shape
        mat = torch.arange(12, dtype=torch.float64).view(3, 4) + 100 * rank
        col = mat[:, 1:3].contiguous()
        into = torch.empty(3, 2, dtype=torch.float64)
        peer = (rank + 1) % world
        source = (rank - 1) % world
        work = sparse_exchange({peer: col}, {source: into}, g, comm, async_op=True)
        work.wait()
        assert_close(into, (torch.arange(12, dtype=torch.float64).view(3, 4) + 100 * source)[:, 1:3], f"{comm}: async exchange", 0, 0)
        # empty tables on every rank are a no-op
        assert sparse_exchange({}, {}, g, comm) is None
        for direction in (1, -1):
            got, work = ring_shift(torch.full((2, 3), float(rank)), None, direction, g, comm)
            assert work is None and torch.all(got == (rank - direction) % world)
            buf = torch.empty(2, 3)
            got, work = ring_shift(torch.full((2, 3), float(rank)), buf, direction, g, comm, async_op=True)
            work.wait()
            assert got is buf and torch.all(buf == (rank - direction) % world)
    assert all_reduce_max(rank * 1.5, g) == 1.5 * (world - 1)
    # a ring on a group made just now (no earlier traffic on it), and on a sub-group with its own numbering
    mesh = jb.make_process_mesh({"a": 2, "b": world // 2})
    sub = mesh["b"]
    got, _ = ring_shift(torch.tensor([float(rank)]), None, 1, sub, CommOp.ISEND)
    want = dist.get_process_group_ranks(sub)[(sub.rank() - 1) % sub.size()]
    assert float(got) == want
    solo = mesh["a"] if world == 2 else None
    if solo is not None and solo.size() == 1:
        got, work = ring_shift(torch.tensor([3.0]), None, 1, solo)
        assert float(got) == 3.0 and work is None


@pytest.mark.parametrize("world", [2, 4])
def test_sparse_exchange_and_ring_shift(world):
    run_distributed(_worker_exchange, world, timeout=300)


def test_backend_names_that_are_accepted_and_refused(monkeypatch):
    """The backend check reads the group's backend string: plain names, the per-device form of a group that runs
    gloo on the CPU and NCCL on the GPUs, and anything else (which would take the NCCL code paths and hang)."""
    import torch.distributed as dist
    from jigsaw_b200._core import comm

    for name, want in (("gloo", {"gloo"}), ("nccl", {"nccl"}), ("cpu:gloo,cuda:nccl", {"gloo", "nccl"})):
        monkeypatch.setattr(dist, "get_backend", lambda group=None, name=name: name)
        assert comm.check_backend() == want
    monkeypatch.setattr(dist, "get_backend", lambda group=None: "gloo")
    assert comm.get_device_of_process_group() == torch.device("cpu")
    for name in ("mpi", "ucc", "cpu:gloo,cuda:ucc"):
        monkeypatch.setattr(dist, "get_backend", lambda group=None, name=name: name)
        with pytest.raises(RuntimeError, match="unsupported process-group backend"):
            comm.check_backend()
