"""Run a function on N ranks (child processes, gloo on CPU or nccl on GPUs) and fail the
test if any rank fails.  Every rank reports through a queue, so a failing rank can never
leave the others (or the test) hanging silently: the parent enforces a timeout and kills
exactly the children it started.

The parity helpers mirror the layout rules of the library: ``split`` cuts a global tensor
by a ``{dim: group}`` spec, ``merge`` gathers it back, ``all_ok`` reduces a verdict so all
ranks agree before asserting.
"""

from __future__ import annotations

import os
import tempfile
import traceback
from collections.abc import Callable
from typing import Any

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _entry(rank: int, world: int, init_file: str, backend: str, fn: Callable, args: tuple, queue: Any) -> None:
    # a rank that is still running after this long prints the stacks of all its threads (to the test's stderr):
    # the place where a hung collective or a lost message blocks is then in the log instead of a bare timeout
    import faulthandler

    faulthandler.enable()            # a crash in native code prints the Python stack of the rank that died
    faulthandler.dump_traceback_later(float(os.environ.get("JIGSAW_TEST_STACKS_AFTER", "90")), exit=False)
    try:
        os.environ["RANK"], os.environ["WORLD_SIZE"], os.environ["LOCAL_RANK"] = str(rank), str(world), str(rank)
        torch.set_num_threads(1)
        # a rank forked from the server inherits its generators: seed them afresh, as a newly started interpreter does,
        # so that ranks which forget to seed do differ from each other
        import random
        import sys

        torch.seed()
        random.seed()
        if "numpy" in sys.modules:
            sys.modules["numpy"].random.seed()
        if backend == "nccl":
            torch.cuda.set_device(rank)
            dist.init_process_group("nccl", init_method=f"file://{init_file}", rank=rank, world_size=world,
                                    device_id=torch.device("cuda", rank))
        else:
            dist.init_process_group("gloo", init_method=f"file://{init_file}", rank=rank, world_size=world)
        fn(rank, world, *args)
        if backend == "nccl":
            torch.cuda.synchronize()
        dist.barrier()
        faulthandler.cancel_dump_traceback_later()
        queue.put((rank, None))
    except BaseException:  # noqa: BLE001 - report everything to the parent
        queue.put((rank, traceback.format_exc()))
    finally:
        try:
            if dist.is_initialized():
                dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass


def _context(backend: str) -> Any:
    """How the ranks are started.  CPU ranks come from a fork server that has imported ``torch`` once (importing it
    costs a rank about three seconds, most of a small test's run time); the server has run nothing, so its children
    start from a clean state, and the library itself is imported by each rank (some tests set switches that are
    read at import).  GPU ranks are spawned: a CUDA context must never be inherited.  ``JIGSAW_TEST_START=spawn``
    spawns the CPU ranks as well."""
    method = os.environ.get("JIGSAW_TEST_START", "spawn" if backend == "nccl" else "forkserver")
    ctx = mp.get_context(method)
    if method == "forkserver":
        ctx.set_forkserver_preload(["torch", "torch.distributed"])
    return ctx


def run_distributed(fn: Callable, world: int, *args: Any, backend: str = "gloo", timeout: float = 240.0) -> None:
    """Spawn ``world`` ranks running ``fn(rank, world, *args)``; raise if any rank raised."""
    ctx = _context(backend)
    queue = ctx.Queue()
    with tempfile.TemporaryDirectory() as tmp:
        init_file = os.path.join(tmp, "rendezvous")
        procs = [ctx.Process(target=_entry, args=(r, world, init_file, backend, fn, args, queue)) for r in range(world)]
        for p in procs:
            p.start()
        results: dict[int, str | None] = {}
        try:
            import queue as _q

            import time

            deadline = time.monotonic() + timeout
            died = None
            while len(results) < world and time.monotonic() < deadline:
                try:
                    rank, err = queue.get(timeout=2.0)
                except _q.Empty:
                    # a rank that died in native code never reports: do not wait for the timeout
                    dead = [(i, p.exitcode) for i, p in enumerate(procs) if p.exitcode not in (None, 0) and i not in results]
                    if dead:
                        died = dead
                        break
                    continue
                results[rank] = err
                if err is not None:
                    break
        finally:
            for p in procs:
                p.join(timeout=10 if len(results) == world and all(v is None for v in results.values()) else 1)
            for p in procs:
                if p.is_alive():
                    p.terminate()
                    p.join(timeout=5)
    errors = {r: e for r, e in results.items() if e is not None}
    if not errors and died:
        raise AssertionError(f"ranks died without reporting (rank, exit code): {died}")
    if errors:
        rank, err = sorted(errors.items())[0]
        raise AssertionError(f"rank {rank} failed:\n{err}")
    if len(results) < world:
        raise AssertionError(f"timeout: only ranks {sorted(results)} of {world} finished within {timeout}s")


# ----------------------------------------------------------------------------- parity helpers
def split(x: torch.Tensor, spec: dict[int, dist.ProcessGroup | None]) -> torch.Tensor:
    """This rank's block of a global tensor: ``spec`` maps a dimension to the group splitting it."""
    for dim, g in spec.items():
        if g is None or g.size() == 1:
            continue
        n = x.shape[dim] // g.size()
        x = x.narrow(dim, g.rank() * n, n)
    return x.contiguous().clone()


def merge(x: torch.Tensor, spec: dict[int, dist.ProcessGroup | None]) -> torch.Tensor:
    """Inverse of :func:`split` (collective)."""
    for dim, g in reversed(list(spec.items())):
        if g is None or g.size() == 1:
            continue
        parts = [torch.empty_like(x) for _ in range(g.size())]
        dist.all_gather(parts, x.contiguous(), group=g)
        x = torch.cat(parts, dim=dim)
    return x


def all_ok(ok: bool) -> bool:
    """MIN-reduce a verdict over the world so that every rank fails together."""
    t = torch.tensor([1 if ok else 0], dtype=torch.int32)
    if dist.get_backend() == "nccl":
        t = t.cuda()
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    return bool(t.item())


def assert_close(a: torch.Tensor, b: torch.Tensor, what: str, rtol: float = 1e-4, atol: float = 1e-5) -> None:
    """Collective assert: all ranks raise if any rank sees a mismatch."""
    ok = a.shape == b.shape and torch.allclose(a.double(), b.double().to(a.device), rtol=rtol, atol=atol)
    detail = ""
    if not ok and a.shape == b.shape:
        detail = f" max abs diff {(a.double() - b.double().to(a.device)).abs().max().item():.3e}"
    elif not ok:
        detail = f" shapes {tuple(a.shape)} vs {tuple(b.shape)}"
    if not all_ok(ok):
        raise AssertionError(f"{what}: mismatch on some rank (rank {dist.get_rank()}: ok={ok}{detail})")


def singleton_mesh(*axes):
    """``{axis: group holding only this rank}`` plus "model" (collective: every rank creates
    the singleton groups of all ranks in the same order)."""
    import torch.distributed as dist

    mine = None
    for r in range(dist.get_world_size()):
        g = dist.new_group([r])
        if r == dist.get_rank():
            mine = g
    return {a: mine for a in (*axes, "model")}
