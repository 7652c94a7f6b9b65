"""Input pipeline for domain-parallel training: tile datasets, replica-keyed sampling and a
pinned-memory device prefetcher.

* :class:`TileDataset` returns this rank's *tile* of each sample, read straight from a
  memory-mapped ``.npy`` file, so I/O per rank shrinks with the number of tiles and no rank
  ever holds a whole sample.
* :func:`replica_sampler` keys the shuffling by the data-parallel index: the ranks of one
  model copy draw the same samples in the same order (their tiles belong together), different
  copies draw different ones, and ``drop_last`` keeps the step count equal (every step has
  collectives).
* :class:`DevicePrefetcher` stages every batch in pinned host memory and copies it on a side
  stream while the previous step computes; the consumer waits on an event, not on the host.

Reference parity: the tile dataset and the dp-keyed ``DistributedSampler`` of
examples/dataloader.py:49-106; the prefetcher has no counterpart there.
"""

from __future__ import annotations

from collections.abc import Iterable, Iterator, Mapping
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist
from torch.utils.data import Dataset, DistributedSampler


class TileDataset(Dataset):
    """Samples ``(N, d0, d1, ...)`` in one ``.npy`` file; ``splits`` maps a *sample* dimension
    (0 = ``d0``) to the process group that cuts it.  ``__getitem__`` returns ``(tile, index)``."""

    def __init__(self, path: str | Path, splits: Mapping[int, dist.ProcessGroup | None]) -> None:
        self.path = Path(path)
        header = np.load(self.path, mmap_mode="r")
        self.n, sample_shape = header.shape[0], header.shape[1:]
        self.window: list[slice] = [slice(None)] * len(sample_shape)
        for dim, group in splits.items():
            if group is None or group.size() == 1:
                continue
            if sample_shape[dim] % group.size():
                raise ValueError(f"sample dimension {dim} of size {sample_shape[dim]} does not split {group.size()} ways")
            n = sample_shape[dim] // group.size()
            self.window[dim] = slice(group.rank() * n, (group.rank() + 1) * n)
        self._array = None                       # opened lazily: one handle per loader worker
        del header

    def __len__(self) -> int:
        return self.n

    def __getitem__(self, i: int) -> tuple[torch.Tensor, int]:
        if self._array is None:
            self._array = np.load(self.path, mmap_mode="r")
        tile = np.ascontiguousarray(self._array[(i, *self.window)])
        return torch.from_numpy(tile), i


def replica_sampler(dataset: Dataset, mesh: Mapping[str, dist.ProcessGroup], dp_key: str = "dp", shuffle: bool = True,
                    seed: int = 0) -> DistributedSampler:
    """``DistributedSampler`` over the data-parallel axis (not the world): call
    ``sampler.set_epoch(e)`` every epoch as usual."""
    dp = mesh.get(dp_key) if hasattr(mesh, "get") else mesh[dp_key]
    replicas, index = (1, 0) if dp is None else (dp.size(), dp.rank())
    return DistributedSampler(dataset, num_replicas=replicas, rank=index, shuffle=shuffle, seed=seed, drop_last=True)


class DevicePrefetcher:
    """Iterate ``loader`` ``depth - 1`` batches ahead: host batch -> pinned staging buffers -> device copy on
    a side stream.  Yields tuples of device tensors that are safe to use on the current stream.
    On a CPU device it just forwards the batches.

    ``reuse_buffers=True`` copies into a fixed ring of ``depth + 1`` device buffers per tensor instead of
    allocating fresh device tensors per batch: no allocator traffic in the loop (large batches otherwise
    make the caching allocator grow, which synchronises the device).  A yielded tensor is then valid until
    ``depth`` further batches have been drawn; clone what must live longer."""

    def __init__(self, loader: Iterable, device: torch.device | str, depth: int = 2, reuse_buffers: bool = False) -> None:
        self.loader, self.device, self.depth = loader, torch.device(device), max(1, depth)
        self.reuse_buffers = reuse_buffers
        self.bytes_copied = 0
        self._pinned: list[list[torch.Tensor]] = []
        self._device: list[list[torch.Tensor]] = []
        self._consumed: list["torch.cuda.Event | None"] = []
        self._stream = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None

    def _to_device(self, slot: int, j: int, src: torch.Tensor) -> torch.Tensor:
        """Device copy of the pinned tensor ``src`` (on the side stream, which is current)."""
        if not self.reuse_buffers:
            return src.to(self.device, non_blocking=True)
        ring = self._device[slot]
        while len(ring) <= j:
            ring.append(None)
        if ring[j] is None or ring[j].shape != src.shape or ring[j].dtype != src.dtype:
            ring[j] = torch.empty(src.shape, dtype=src.dtype, device=self.device)
        ring[j].copy_(src, non_blocking=True)
        return ring[j]

    def _stage(self, slot: int, batch) -> tuple[tuple[torch.Tensor, ...], "torch.cuda.Event | None", int]:
        tensors = tuple(batch) if isinstance(batch, (tuple, list)) else (batch,)
        if self._stream is None:
            return tuple(t if not torch.is_tensor(t) else t.to(self.device) for t in tensors), None, slot
        while len(self._pinned) <= slot:
            self._pinned.append([])
            self._device.append([])
            self._consumed.append(None)
        stage = self._pinned[slot]
        out = []
        if self.reuse_buffers and self._consumed[slot] is not None:
            self._stream.wait_event(self._consumed[slot])   # the consumer's work on this slot's previous batch
        with torch.cuda.stream(self._stream):
            for j, t in enumerate(tensors):
                if not torch.is_tensor(t):
                    out.append(t)
                    continue
                if t.is_pinned():                      # already page-locked: copy straight from it
                    while len(stage) <= j:
                        stage.append(t)
                    out.append(self._to_device(slot, j, t))
                    self.bytes_copied += t.numel() * t.element_size()
                    continue
                if j >= len(stage) or stage[j].shape != t.shape or stage[j].dtype != t.dtype:
                    buf = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
                    stage[j:j + 1] = [buf]
                stage[j].copy_(t)
                out.append(self._to_device(slot, j, stage[j]))
                self.bytes_copied += t.numel() * t.element_size()
            ready = torch.cuda.Event()
            ready.record(self._stream)
        return tuple(out), ready, slot

    def __iter__(self) -> Iterator[tuple[torch.Tensor, ...]]:
        queue: list = []
        slot = 0
        for batch in self.loader:
            queue.append(self._stage(slot % (self.depth + 1), batch))
            slot += 1
            if len(queue) > self.depth - 1:
                yield from self._hand_out(queue.pop(0))
        while queue:
            yield from self._hand_out(queue.pop(0))

    def _hand_out(self, item) -> Iterator[tuple[torch.Tensor, ...]]:
        tensors, ready, slot = item
        if ready is None:
            yield tensors
            return
        current = torch.cuda.current_stream(self.device)
        current.wait_event(ready)
        if not self.reuse_buffers:
            for t in tensors:
                if torch.is_tensor(t):
                    t.record_stream(current)
        yield tensors
        if self.reuse_buffers:      # back from the consumer: everything it did with this batch is queued by now
            done = torch.cuda.Event()
            done.record(torch.cuda.current_stream(self.device))
            self._consumed[slot] = done
