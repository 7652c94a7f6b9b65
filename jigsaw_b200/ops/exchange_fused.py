"""Re-sharding all-to-all over peer memory (``csrc/alltoall.cu``): split one dimension over the
ranks of a group and concatenate what arrives along another, in one kernel that stores every
vector at its final place in the destination rank's output.  This is the sequence <-> head
exchange of Ulysses attention (and its inverse, which is also its backward).

Reference parity: ``all_to_all_single`` in
jigsaw/modules/attention/_functional/ulysses.py:40,63 (NCCL there, plus the permutes around it).
"""

from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from . import _lib, symm

_HEADER = 256
_side_streams: dict[int, "torch.cuda.Stream"] = {}


def _ring_block(ar: "symm.PeerArena", tag: tuple, nbytes: int) -> "symm.Block":
    """The next block of the two-deep staging ring ``tag`` (:meth:`symm.PeerArena.ring_block`)."""
    return ar.ring_block(tag, nbytes)


@_lib.traced("jb.maybe_fused_all_to_all")
@_lib.audited("all_to_all")
def maybe_fused_all_to_all(x: torch.Tensor, group: dist.ProcessGroup, split_dim: int, cat_dim: int) -> torch.Tensor | None:
    """``cat(all_to_all(chunks of x along split_dim), dim=cat_dim)`` or ``None`` when the kernel
    does not apply (needs a contiguous CUDA tensor whose trailing dimensions behind both
    ``split_dim`` and ``cat_dim`` make up a multiple of 16 bytes)."""
    nd = x.dim()
    s, c = split_dim % nd, cat_dim % nd
    P = group.size()
    if not x.is_cuda or P < 2 or P > 8 or s == c or x.numel() == 0 or x.shape[s] % P:
        return None
    last = max(s, c)
    tail = 1
    for n in x.shape[last + 1:]:
        tail *= n
    if (tail * x.element_size()) % 16 or torch._C._functorch.is_batchedtensor(x) or not _lib.available():
        return None
    # collapse to [D0][D1][D2][D3][V]: before first, first, between, second, tail
    first, second = min(s, c), last
    d0 = 1
    for n in x.shape[:first]:
        d0 *= n
    mid = 1
    for n in x.shape[first + 1:second]:
        mid *= n
    dims = [d0, x.shape[first], mid, x.shape[second], tail * x.element_size() // 16]
    split, cat = (1, 3) if s < c else (3, 1)
    x = x.contiguous()
    dev = x.device
    ar = symm.arena(dev)
    L = _lib.lib()
    me = group.rank()
    ranks = dist.get_process_group_ranks(group)
    nbytes = x.numel() * x.element_size()
    blk = _ring_block(ar, ("a2a", dev.index, nbytes, tuple(ranks)), _HEADER + nbytes)
    epoch = ar.next_own_epoch(blk)
    a = _lib.JbA2a()
    a.x = x.data_ptr()
    for i, n in enumerate(dims):
        a.dim[i] = n
    a.split, a.cat, a.parts, a.me = split, cat, P, me
    for i, r in enumerate(ranks):
        a.out[i] = (blk.ptr if i == me else blk.peer_ptr(r)) + _HEADER
        a.flag_out[i] = None if i == me else blk.peer_ptr(r) + 4 * me
        a.flag_in[i] = None if i == me else blk.ptr + 4 * i
    a.epoch = epoch
    if ar.capture_stride is not None:
        a.stride, a.replay = ar.capture_stride, ar.replay.data_ptr()
    rc = L.jb_all_to_all(ctypes.byref(a), ctypes.c_void_p(ar.done_counter.data_ptr()), ctypes.c_void_p(ar.status.data_ptr()),
                         _lib.sm_count(dev.index), _lib.stream_ptr())
    if rc != 0:
        raise RuntimeError(f"jigsaw_b200 kernel launcher all_to_all failed with code {rc}")
    _lib.count_launches(1)
    shape = list(x.shape)
    shape[s] //= P
    shape[c] *= P
    return blk.tensor[_HEADER:_HEADER + nbytes].view(x.dtype).view(shape).clone()


class PeerChunks:
    """A tensor that every rank of ``group`` publishes once in symmetric memory and whose copies the
    others fetch on demand, straight from the owner's memory (ring attention's key / value chunks).

    ``PeerChunks(payload, group)`` stages the local payload and publishes its epoch flag to the
    peers; ``fetch(owner)`` returns a local copy of ``owner``'s payload, pulled by a kernel that
    waits (bounded) for the owner's flag and then reads over NVLink.  Fetches run on a side stream,
    so the next chunk can travel while the current one is being used; the returned tensor is safe
    to use on the current stream."""

    def __init__(self, payload: torch.Tensor, group: dist.ProcessGroup) -> None:
        self.payload = payload.contiguous()
        self.group = group
        dev = payload.device
        self.ar = symm.arena(dev)
        self.me = group.rank()
        self.ranks = dist.get_process_group_ranks(group)
        self.nbytes = self.payload.numel() * self.payload.element_size()
        blk = _ring_block(self.ar, ("chunks", dev.index, self.nbytes, tuple(self.ranks)), _HEADER + self.nbytes)
        self.blk = blk
        staged = blk.tensor[_HEADER:_HEADER + self.nbytes].view(self.payload.dtype).view(self.payload.shape)
        staged.copy_(self.payload)
        self.epoch = self.ar.next_own_epoch(blk)
        self.stride = self.ar.capture_stride or 0
        self.replay = self.ar.replay.data_ptr() if self.ar.capture_stride is not None else None
        flags = (ctypes.c_void_p * 8)()
        n = 0
        for i, r in enumerate(self.ranks):
            if i != self.me:
                flags[n] = blk.peer_ptr(r) + 4 * self.me
                n += 1
        rc = _lib.lib().jb_publish(flags, n, self.epoch, self.stride, self.replay, _lib.stream_ptr())
        if rc != 0:
            raise RuntimeError(f"jigsaw_b200 kernel launcher publish failed with code {rc}")
        _lib.count_launches(1)
        if dev.index not in _side_streams:
            _side_streams[dev.index] = torch.cuda.Stream(dev)
        self._side = _side_streams[dev.index]
        self._staged_event = torch.cuda.Event()
        self._staged_event.record()

    @staticmethod
    def usable(payload: torch.Tensor, group: dist.ProcessGroup) -> bool:
        nbytes = payload.numel() * payload.element_size()
        return (payload.is_cuda and 2 <= group.size() <= 8 and nbytes % 16 == 0 and nbytes > 0
                and not torch._C._functorch.is_batchedtensor(payload) and _lib.available())

    def start(self, owner: int) -> tuple[torch.Tensor, "torch.cuda.Event | None"]:
        """Begin fetching ``owner``'s payload (group rank); returns ``(buffer, ready event)``."""
        if owner == self.me:
            return self.payload, None
        dev = self.payload.device
        buf = torch.empty_like(self.payload)
        self._side.wait_event(self._staged_event)
        with torch.cuda.stream(self._side):
            src = self.blk.peer_ptr(self.ranks[owner]) + _HEADER
            rc = _lib.lib().jb_peer_fetch(ctypes.c_void_p(src), ctypes.c_void_p(buf.data_ptr()), self.nbytes,
                                          ctypes.c_void_p(self.blk.ptr + 4 * owner), self.epoch, self.stride, self.replay,
                                          ctypes.c_void_p(self.ar.status.data_ptr()), 4 * _lib.sm_count(dev.index),
                                          _lib.stream_ptr())
            if rc != 0:
                raise RuntimeError(f"jigsaw_b200 kernel launcher peer_fetch failed with code {rc}")
            ready = torch.cuda.Event()
            ready.record()
        buf.record_stream(self._side)
        _lib.count_launches(1)
        return buf, ready
