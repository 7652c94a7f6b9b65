"""Asynchronous activation offload to pinned host memory and back.

Device-to-host copies run on a side stream; the consumer prefetches the next chunk
host-to-device while computing on the current one.  Events, never host waits, order the
copies against the compute stream.

Reference parity: jigsaw/_core/offload.py:6-93 (NVLinkActivationOffloader).
"""

from __future__ import annotations

import torch


class ActivationOffloader:
    """Offload tensors to pinned CPU memory on a side stream and fetch them back."""

    def __init__(self, device: torch.device | str) -> None:
        self.device = torch.device(device)
        self.enabled = self.device.type == "cuda"
        self.stream = torch.cuda.Stream(device=self.device) if self.enabled else None
        self._pending: list[torch.cuda.Event] = []

    def offload(self, t: torch.Tensor) -> torch.Tensor:
        """Start copying ``t`` to the host; returns the (pinned) host tensor."""
        if not self.enabled:
            return t
        host = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True)
        ready = torch.cuda.Event()
        ready.record(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self.stream):
            self.stream.wait_event(ready)
            host.copy_(t, non_blocking=True)
            done = torch.cuda.Event()
            done.record(self.stream)
        t.record_stream(self.stream)
        self._pending.append(done)
        return host

    def wait_offloads(self) -> None:
        """Make the compute stream wait for every copy started so far (frees the sources)."""
        if not self.enabled:
            return
        cur = torch.cuda.current_stream(self.device)
        for ev in self._pending:
            cur.wait_event(ev)
        self._pending.clear()

    def prefetch(self, host: torch.Tensor) -> tuple[torch.Tensor, "torch.cuda.Event | None"]:
        """Start copying ``host`` back; returns ``(device tensor, event to wait on)``."""
        if not self.enabled or host.device.type != "cpu":
            return host, None
        for ev in self._pending:
            self.stream.wait_event(ev)
        with torch.cuda.stream(self.stream):
            dev = host.to(self.device, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.stream)
        return dev, ev

    def consume(self, dev: torch.Tensor, ev: "torch.cuda.Event | None") -> torch.Tensor:
        """Order the compute stream after the prefetch of ``dev`` and return it."""
        if ev is not None:
            torch.cuda.current_stream(self.device).wait_event(ev)
            dev.record_stream(torch.cuda.current_stream(self.device))
        return dev


NVLinkActivationOffloader = ActivationOffloader
