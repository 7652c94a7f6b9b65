"""Device-side timing and profiler ranges.

:class:`DeviceTimer` brackets a region with CUDA events on the current stream and reports
the maximum over the ranks of a group (a multi-GPU step takes as long as its slowest rank);
:func:`nvtx_range` marks a region for Nsight tools and is free when no profiler is attached.

Reference parity: the reference times on the host (``jigsaw/log.py`` ``timed``); the device
timer is the B200-side replacement used by ``bench.py``.
"""

from __future__ import annotations

import contextlib
from collections.abc import Iterator

import torch
import torch.distributed as dist


class DeviceTimer:
    def __init__(self, device: torch.device | str | None = None, group: dist.ProcessGroup | None = None) -> None:
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.group = group
        self._start = torch.cuda.Event(enable_timing=True)
        self._stop = torch.cuda.Event(enable_timing=True)
        self.ms: float | None = None

    def __enter__(self) -> "DeviceTimer":
        if dist.is_initialized():
            dist.barrier(group=self.group)
        torch.cuda.synchronize(self.device)
        self._start.record()
        return self

    def __exit__(self, *exc) -> None:
        self._stop.record()
        torch.cuda.synchronize(self.device)
        ms = torch.tensor([self._start.elapsed_time(self._stop)], device=self.device)
        if dist.is_initialized():
            dist.all_reduce(ms, op=dist.ReduceOp.MAX, group=self.group)
        self.ms = float(ms.item())


@contextlib.contextmanager
def nvtx_range(name: str) -> Iterator[None]:
    if torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield
