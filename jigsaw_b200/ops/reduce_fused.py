"""Gradient all-reduce on an own kernel over peer memory, optionally hidden under the backward pass.

``maybe_fused_all_reduce(tensors, ranks)`` sums fp32 tensors in place over the GPUs ``ranks`` (world
ranks, this one included) with ONE kernel launch per rank (``csrc/allreduce.cu``: staged / done notices,
reduce-scatter by peer loads, all-gather by peer stores) instead of a library collective; the tensors
are packed into, and unpacked from, a symmetric staging buffer by one multi-tensor copy each.

:class:`OverlappedReducer` does the same on a side stream: ``add()`` is called as soon as a layer's
weight gradient has been launched, the reduction then runs while the remaining data- and
weight-gradient kernels of the backward pass occupy the GPU, and ``finish()`` joins the side stream
before the optimizer.  The result is bit-identical on every rank (each element is summed by exactly one
rank, in rank order) and independent of timing.

Reference parity: the blocking flat all-reduce of jigsaw/parallel/_sync.py:19-53 and the bucket hook of
jigsaw/parallel/_joint.py:215-279, both on NCCL there.
"""

from __future__ import annotations

import ctypes
from collections.abc import Sequence
from typing import Any

import torch
import torch.distributed as dist

from . import _lib, symm

_HEADER = 256
_MAX_BLOCKS = 32
_blocks: dict[tuple, Any] = {}
_counters: dict[tuple, torch.Tensor] = {}
_side: dict[int, torch.cuda.Stream] = {}


def _size_class(nbytes: int) -> int:
    c = 16384
    while c < nbytes:
        c *= 2
    return c


def usable(tensors: Sequence[torch.Tensor], ranks: Sequence[int]) -> bool:
    if not tensors or not 2 <= len(ranks) <= 8 or not dist.is_initialized():
        return False
    return all(t.is_cuda and t.dtype == torch.float32 and not torch._C._functorch.is_batchedtensor(t) for t in tensors) \
        and _lib.available()


def _launch(tensors: Sequence[torch.Tensor], ranks: Sequence[int], scale: float, lane: str) -> None:
    """Pack, reduce and unpack on the current stream."""
    dev = tensors[0].device
    ar = symm.arena(dev)
    ranks = sorted(int(r) for r in ranks)
    me = ranks.index(dist.get_rank())
    n = sum(t.numel() for t in tensors)
    n4 = (n + 3) // 4 * 4
    cls = _size_class(n4 * 4)
    key = (lane, dev.index, cls, tuple(ranks))
    blk = _blocks.get(key)
    if blk is None:
        blk = _blocks[key] = ar.alloc(_HEADER + cls, tag=("allreduce",) + key)
        _counters[key] = torch.zeros(1, dtype=torch.int32, device=dev)
    flat = blk.tensor[_HEADER:_HEADER + n4 * 4].view(torch.float32)
    views, off = [], 0
    for t in tensors:
        views.append(flat[off:off + t.numel()].view(t.shape))
        off += t.numel()
    if n4 != n:
        flat[n:].zero_()
    torch._foreach_copy_(views, [t.detach() for t in tensors])
    r = _lib.JbAllReduce()
    for i, w in enumerate(ranks):
        r.buf[i] = (blk.ptr if i == me else blk.peer_ptr(w)) + _HEADER
        r.notice_out[i] = None if i == me else blk.peer_ptr(w) + 4 * me
        r.notice_in[i] = None if i == me else blk.ptr + 4 * i
    r.epoch = ar.next_own_epoch(blk)
    r.stride = ar.capture_stride or 0
    r.replay = ar.replay.data_ptr() if ar.capture_stride is not None else None
    r.ranks, r.me, r.n, r.scale = len(ranks), me, n4, float(scale)
    rc = _lib.lib().jb_all_reduce_sum(ctypes.byref(r), ctypes.c_void_p(_counters[key].data_ptr()),
                                      ctypes.c_void_p(ar.status.data_ptr()), _MAX_BLOCKS, _lib.stream_ptr())
    if rc != 0:
        raise RuntimeError(f"jigsaw_b200 kernel launcher all_reduce_sum failed with code {rc}")
    _lib.count_launches(1)
    torch._foreach_copy_([t.detach() for t in tensors], views)


@_lib.traced("jb.maybe_fused_all_reduce")
@_lib.audited("all_reduce")
def maybe_fused_all_reduce(tensors: Sequence[torch.Tensor], ranks: Sequence[int], scale: float = 1.0) -> bool | None:
    """In place ``t <- scale * sum over ranks of t`` for every fp32 CUDA tensor of ``tensors`` on the
    current stream; ``True`` when done, ``None`` when the kernel does not apply (the caller then uses the
    process group's all-reduce)."""
    if not tensors or not tensors[0].is_cuda:
        return None
    if not usable(tensors, ranks):
        return _lib.decline("needs fp32 CUDA tensors and a group of 2 to 8 ranks")
    _launch(tensors, ranks, scale, "main")
    return True


class OverlappedReducer:
    """Sums gradients over ``ranks`` on a side stream while the caller keeps launching backward kernels.

        red = OverlappedReducer(device, ranks)
        ...                       # launch the kernels that produce gw, gb
        red.add([gw, gb])         # reduction starts once they are complete, on the side stream
        ...                       # more backward kernels
        red.finish()              # the current stream waits for every pending reduction
    """

    def __init__(self, device: torch.device, ranks: Sequence[int], scale: float = 1.0) -> None:
        self.device, self.ranks, self.scale = device, list(ranks), scale
        idx = device.index if device.index is not None else torch.cuda.current_device()
        if idx not in _side:
            _side[idx] = torch.cuda.Stream(device)
        self.side = _side[idx]
        self.pending = False

    def add(self, tensors: Sequence[torch.Tensor]) -> None:
        ready = torch.cuda.Event()
        ready.record()
        self.side.wait_event(ready)
        with torch.cuda.stream(self.side):
            _launch(tensors, self.ranks, self.scale, "side")
        self.pending = True          # the tensors stay alive until finish(): no allocator bookkeeping needed

    def finish(self) -> None:
        if self.pending:
            done = torch.cuda.Event()
            done.record(self.side)
            torch.cuda.current_stream(self.device).wait_event(done)
            self.pending = False
