"""Peer-memory runtime: symmetric buffers, flag slots and neighbour tables for the fused kernels.

Every rank of the job allocates the same sequence of blocks from a :class:`PeerArena`, so a
block has the same offset on every rank and a kernel can address a neighbour's copy as
``peer_base[rank] + offset``.  The arena grows in segments; each segment is one symmetric
allocation (``torch.distributed._symmetric_memory``: CUDA VMM allocation plus handle
exchange over the process group), so growing is a collective that all ranks reach together
because they run the same program.  Blocks are recycled through exact-size free lists, which
keeps the allocation sequence deterministic across ranks.

Signalling: each padded buffer owns a *slot* of 16 flag words in a small symmetric flag
segment.  A producer kernel publishes a monotonically increasing epoch into the slot of each
neighbour once its peer stores are visible; a consumer kernel waits (bounded) until the flags
of all its neighbours reach the epoch.  With one rank, no symmetric memory is used at all.

Reference parity: the reference has no peer-memory layer; it moves halos with
``all_to_all_single`` (jigsaw/modules/convolution/_common/halo.py:7-63).  This module is the
B200-native replacement of that transport.
"""

from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from ._lib import JbHalo

_ALIGN = 1024
_FLAG_WORDS = 32           # words 0..8: halo arrival per direction; words 16..24: release acknowledgements
_ACK_BASE = 16
_MAX_SLOTS = 4096


def _round_up(n: int, a: int) -> int:
    return (n + a - 1) // a * a


class Block:
    """A sub-range of the arena: same offset on every rank."""

    __slots__ = ("arena", "segment", "offset", "nbytes", "slot", "epoch", "tensor", "tag", "own_epoch", "readers")

    def __init__(self, arena: "PeerArena", segment: int, offset: int, nbytes: int, tensor: torch.Tensor) -> None:
        self.arena, self.segment, self.offset, self.nbytes = arena, segment, offset, nbytes
        self.tensor = tensor
        self.slot = -1
        self.epoch = 0
        self.own_epoch = 0          # epoch of flags that live inside the block itself
        self.tag: object = None
        self.readers: list | None = None   # neighbour table of the last halo production, until released

    @property
    def ptr(self) -> int:
        return self.tensor.data_ptr()

    def peer_ptr(self, world_rank: int) -> int:
        return self.arena.peer_base(self.segment, world_rank) + self.offset

    def check_range(self, offset: int, nbytes: int, pitch: int = 0, rows: int = 1) -> None:
        """Raise unless ``rows`` pieces of ``nbytes`` bytes, ``pitch`` bytes apart, starting ``offset`` bytes into
        the block, lie inside it.  Every copy into a peer's copy of a block is checked with this on the host before
        it is enqueued: an address outside the block would land in whatever the peer keeps next to it."""
        last = offset + (rows - 1) * pitch + nbytes
        if offset < 0 or nbytes <= 0 or rows < 1 or (rows > 1 and pitch < nbytes) or last > self.nbytes:
            raise ValueError(f"range (offset {offset}, {rows} x {nbytes} bytes, pitch {pitch}) does not fit a block of {self.nbytes} bytes")

    def view(self, shape: tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        return self.tensor.view(dtype)[: int(torch.Size(shape).numel())].view(shape)


class PeerArena:
    """Symmetric block allocator shared by all ranks of the default process group."""

    def __init__(self, device: torch.device) -> None:
        self.device = device
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.symmetric = self.world > 1
        self._segments: list[dict] = []
        self._free: dict[tuple, list[Block]] = {}
        self._free_slots = list(range(_MAX_SLOTS - 1, -1, -1))
        self._slot_epoch = [0] * _MAX_SLOTS
        self.done_counter = torch.zeros(4, dtype=torch.int32, device=device)
        self.status = torch.zeros(4, dtype=torch.int32, device=device)
        # CUDA-graph support: kernels inside a captured step take their epochs as
        # ``captured value + replays * productions of the slot per step`` (see begin_capture)
        self.replay = torch.zeros(1, dtype=torch.int32, device=device)
        # epoch of the latest content produced into each flag slot, kept on the device (see acquire())
        self.last_epoch = torch.zeros(_MAX_SLOTS, dtype=torch.int32, device=device)
        self._capture_stride: int | None = None
        self._capture_slots: set[int] = set()
        self._capture_blocks: list[Block] = []
        self._rings: dict[tuple, list] = {}
        self._ring_uses: dict[tuple, int] = {}
        self._flags = None
        if self.symmetric:
            self._flags = self._new_symmetric(_MAX_SLOTS * _FLAG_WORDS * 4)
            self._flags["tensor"].zero_()
            torch.cuda.synchronize(device)
            dist.barrier()

    # ------------------------------------------------------------------ segments
    def _new_symmetric(self, nbytes: int) -> dict:
        import torch.distributed._symmetric_memory as symm_mem

        t = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
        handle = symm_mem.rendezvous(t, group=dist.group.WORLD)
        return {"tensor": t, "handle": handle, "ptrs": [int(p) for p in handle.buffer_ptrs], "used": 0, "size": nbytes}

    def _new_segment(self, at_least: int) -> int:
        default = int(float(os.environ.get("JIGSAW_B200_ARENA_SEGMENT_GB", "1")) * (1 << 30))
        nbytes = _round_up(max(at_least, default), 1 << 21)
        if self.symmetric:
            seg = self._new_symmetric(nbytes)
        else:
            t = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
            seg = {"tensor": t, "handle": None, "ptrs": [t.data_ptr()], "used": 0, "size": nbytes}
        self._segments.append(seg)
        return len(self._segments) - 1

    def reserve(self, nbytes: int) -> None:
        """Make sure a segment with ``nbytes`` of free room exists (collective over the world, like every growth
        of the arena: mapping a segment into the peers is a rendezvous).  Growth happens when a request finds
        no room, which is the same moment on every rank as long as all ranks issue the same sequence of
        requests; a program whose ranks may diverge (data-dependent shapes, ranks that skip a layer) should
        reserve its peak here, at a point all ranks pass, so that no later request has to grow."""
        size = _round_up(nbytes, _ALIGN)
        if any(seg["size"] - seg["used"] >= size for seg in self._segments):
            return
        i = self._new_segment(size)
        self._segments[i]["tensor"].zero_()
        if self.symmetric:
            torch.cuda.synchronize(self.device)
            dist.barrier()

    def peer_base(self, segment: int, world_rank: int) -> int:
        ptrs = self._segments[segment]["ptrs"]
        return ptrs[world_rank if self.symmetric else 0]

    # ------------------------------------------------------------------ blocks
    def alloc(self, nbytes: int, zero: bool = False, tag: object = None) -> Block:
        """A block of at least ``nbytes`` (1 KiB aligned).  A recycled block is only handed to a
        request with the same ``tag`` (callers tag padded buffers with their geometry, so the
        never-written zero border of a recycled buffer is still in the right place) and keeps
        its contents unless ``zero``; fresh segments come zero-filled.  A request that finds no room grows the
        arena, which is collective (see :meth:`reserve`); every other request is local."""
        size = _round_up(nbytes, _ALIGN)
        pool = self._free.get((size, tag))
        if pool:
            blk = pool.pop()
            if zero:
                blk.tensor.zero_()
            return blk
        for i, seg in enumerate(self._segments):
            if seg["size"] - seg["used"] >= size:
                break
        else:
            i = self._new_segment(size)
            self._segments[i]["tensor"].zero_()
            if self.symmetric:
                torch.cuda.synchronize(self.device)
                dist.barrier()
        seg = self._segments[i]
        off = seg["used"]
        seg["used"] += size
        blk = Block(self, i, off, size, seg["tensor"][off : off + size])
        blk.tag = tag
        return blk

    def free(self, blk: Block) -> None:
        """Return ``blk`` to its pool.  Every kernel that reads its content must already be on
        the current stream: if neighbours pushed a halo into it, they are told here (in stream
        order) that its border may be overwritten.  The block keeps its flag slot for good."""
        self.release(blk)
        self._free.setdefault((blk.nbytes, blk.tag), []).append(blk)

    # ------------------------------------------------------------------ write-after-read protection
    def acquire(self, blk: Block, nbrs: list) -> int:
        """Take the next epoch of ``blk`` for a production whose edges go to ``nbrs``.  A tiny
        kernel on the current stream first waits (bounded) until every neighbour has released the
        previous content of its copy of the block: a rank that runs ahead must not push a new
        border into memory that its neighbour's kernels still read."""
        from . import _lib

        self.bind_slot(blk)
        acks = (ctypes.c_void_p * 8)()
        n = 0
        for d, r in enumerate(nbrs):
            if r is not None:
                acks[n] = self.flag_ptr(self.rank, blk.slot, _ACK_BASE + d)
                n += 1
        epoch = self.next_epoch(blk)
        stride = self._capture_stride or 0
        replay = ctypes.c_void_p(self.replay.data_ptr()) if self._capture_stride is not None else None
        rc = _lib.lib().jb_slot_acquire(acks, n, ctypes.c_void_p(self.last_epoch.data_ptr() + 4 * blk.slot), epoch, stride,
                                        replay, ctypes.c_void_p(self.status.data_ptr()), _lib.stream_ptr())
        if rc != 0:
            raise RuntimeError(f"jigsaw_b200 kernel launcher slot_acquire failed with code {rc}")
        _lib.count_launches(1)
        blk.readers = list(nbrs)
        return epoch

    def release(self, blk: Block) -> None:
        """Tell the neighbours that pushed into ``blk`` that its current content has been consumed
        (everything enqueued so far on the current stream).  Idempotent per production."""
        if blk.readers is None or not self.symmetric:
            return
        from . import _lib

        rel = (ctypes.c_void_p * 8)()
        n = 0
        for d, r in enumerate(blk.readers):
            if r is not None:
                rel[n] = self.flag_ptr(r, blk.slot, _ACK_BASE + 8 - d)
                n += 1
        blk.readers = None
        stride = self._capture_stride or 0
        replay = ctypes.c_void_p(self.replay.data_ptr()) if self._capture_stride is not None else None
        try:
            rc = _lib.lib().jb_slot_release(rel, n, blk.epoch, stride, replay, _lib.stream_ptr())
        except Exception:                       # interpreter shutdown: the context may be gone
            return
        if rc != 0:
            raise RuntimeError(f"jigsaw_b200 kernel launcher slot_release failed with code {rc}")
        _lib.count_launches(1)

    # ------------------------------------------------------------------ flags
    def bind_slot(self, blk: Block) -> None:
        if blk.slot < 0:
            blk.slot = self._free_slots.pop()

    def next_epoch(self, blk: Block) -> int:
        """Advance and return the epoch of the block's slot (one per production of its content)."""
        self.bind_slot(blk)
        if self._capture_stride is not None:
            self._capture_slots.add(blk.slot)
        self._slot_epoch[blk.slot] += 1
        blk.epoch = self._slot_epoch[blk.slot]
        return blk.epoch

    def begin_capture(self, stride: int) -> None:
        """From now on halo descriptors refer to the replay counter: a launch captured with
        epoch ``e`` publishes / awaits ``e + replays * stride``.  ``stride`` must exceed the
        number of times any one slot is produced between two replays (captured step plus
        eager steps in between); which buffer gets which slot may differ from step to step,
        so one generous stride serves all slots."""
        self._capture_stride = int(stride)
        self._capture_slots = set()
        self._capture_blocks = []

    def end_capture(self) -> tuple[set[int], list[Block]]:
        """Leave capture mode; returns the flag slots and the self-flagged blocks that the
        captured step produces."""
        self._capture_stride = None
        return set(self._capture_slots), list(self._capture_blocks)

    def advance(self, produced: tuple[set[int], list[Block]], stride: int) -> None:
        """Account on the host for one replay of a captured step."""
        slots, blocks = produced
        for slot in slots:
            self._slot_epoch[slot] += stride
        for blk in blocks:
            blk.own_epoch += stride

    def next_own_epoch(self, blk: Block) -> int:
        """Advance and return the epoch of flags kept inside ``blk`` (blocks are the same on
        every rank, so their counters agree without communication)."""
        blk.own_epoch += 1
        if self._capture_stride is not None and not any(b is blk for b in self._capture_blocks):
            self._capture_blocks.append(blk)
        return blk.own_epoch

    @property
    def capture_stride(self) -> int | None:
        return self._capture_stride

    def ring_block(self, tag: tuple, nbytes: int) -> Block:
        """Two staging blocks per ``tag`` (geometry and ranks of the operation's group, so operations over
        different groups never share a ring), used alternately.  A rank can run at most one such operation
        ahead of its peers (it needs their flag of the current one, which they raise after finishing the
        previous one), so the block it overwrites is never one that a peer may still be reading."""
        ring = self._rings.get(tag)
        if ring is None:
            ring = self._rings[tag] = [[self.alloc(nbytes, tag=tag + (i,)) for i in range(2)], 0]
        blk = ring[0][ring[1] & 1]
        ring[1] += 1
        self._ring_uses[tag] = self._ring_uses.get(tag, 0) + 1
        return blk

    def start_ring_count(self) -> None:
        self._ring_uses = {}

    def some_ring_used_an_odd_number_of_times(self) -> bool:
        """Since :meth:`start_ring_count`.  A step that does so, replayed as a CUDA graph, ends and begins on
        the SAME block of that ring, and the alternation argument of :meth:`ring_block` no longer separates
        the last use of one replay from the first use of the next."""
        return any(n & 1 for n in self._ring_uses.values())

    def flag_ptr(self, world_rank: int, slot: int, direction: int) -> int:
        return self._flags["ptrs"][world_rank] + (slot * _FLAG_WORDS + direction) * 4

    def check_status(self, group: dist.ProcessGroup | None = None, collective: bool = False) -> None:
        """Raise if any kernel recorded a bounded-wait timeout (synchronises the device).  With
        ``collective=True`` (or a ``group``) the code is MAX-reduced first, so that every rank of the
        group raises when any of them saw an error: a rank whose peer never arrived and the peer that
        was late fail together instead of one of them waiting in the next collective."""
        if collective or group is not None:
            code = agree_on_status(self.status[:1], group)
        else:
            code = int(self.status[0].item())
        if code != 0:
            self.status.zero_()
            raise RuntimeError(f"jigsaw_b200 kernel error {code}: {STATUS_NAMES.get(code, 'unknown')}")


STATUS_NAMES = {1: "an mbarrier wait timed out", 2: "a cross-GPU flag wait timed out", 3: "bad argument"}


def agree_on_status(status: torch.Tensor, group: dist.ProcessGroup | None = None) -> int:
    """Largest status code over the ranks of ``group`` (the world when ``None``); ``status`` is a
    one-element integer tensor on the device of the group's backend.  Without a process group it is
    just this rank's code."""
    t = status.detach().clone()
    if dist.is_available() and dist.is_initialized():
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return int(t.item())


_arenas: dict[int, PeerArena] = {}


def arena(device: torch.device) -> PeerArena:
    """The arena of ``device`` (created on first use; collective when the job has several ranks)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _arenas:
        _arenas[idx] = PeerArena(torch.device("cuda", idx))
    return _arenas[idx]


# --------------------------------------------------------------------------- all-gather by push
_push_streams: dict[int, torch.cuda.Stream] = {}
_epoch_words: dict[int, torch.Tensor] = {}


def push_slot_to_peers(ar: "PeerArena", blk: Block, ranks: list, me: int, offset: int, nbytes: int, pitch: int = 0,
                        rows: int = 1) -> tuple:
    """Give every peer this rank's slot of ``blk`` (``nbytes`` at ``offset``, already written locally on the
    current stream) and then raise this rank's flag in the peer's copy of the block.  Both travel by the copy
    engines on a side stream: every staged byte crosses NVLink once per destination, no SM is used, and
    the caller's attention kernel (launched next on the current stream) starts on its own part at once while
    the pushes of all ranks are in flight.  Returns ``(epoch, stride, replay, done event)``; the caller makes
    its stream wait for the event AFTER launching its kernel."""
    from . import _lib

    L, dev = _lib.lib(), blk.tensor.device
    blk.check_range(offset, nbytes, pitch, rows)
    if len(ranks) > 8 or not 0 <= me < len(ranks):
        raise ValueError(f"a staged block is shared by at most 8 ranks and this rank must be one of them (got {len(ranks)}, index {me})")
    epoch = ar.next_own_epoch(blk)
    stride = ar.capture_stride or 0
    replay = ar.replay.data_ptr() if ar.capture_stride is not None else None
    idx = dev.index
    if idx not in _push_streams:
        _push_streams[idx] = torch.cuda.Stream(dev)
        _epoch_words[idx] = torch.zeros(64, dtype=torch.int32, device=dev)
    side = _push_streams[idx]
    # the flag value as it must read on this replay: one word per block (the two blocks of a ring alternate)
    word = _epoch_words[idx][(blk.offset // 1024) % 64:][:1]
    one = (ctypes.c_void_p * 8)()
    one[0] = word.data_ptr()
    rc = L.jb_publish(one, 1, epoch, stride, replay, _lib.stream_ptr())
    staged = torch.cuda.Event()
    staged.record()
    side.wait_event(staged)
    with torch.cuda.stream(side):
        st = _lib.stream_ptr()
        for i, r in enumerate(ranks):
            if i == me or rc != 0:
                continue
            if rows > 1:        # a column block: `rows` pieces of `nbytes`, `pitch` bytes apart
                rc = L.jb_memcpy2d_async(ctypes.c_void_p(blk.peer_ptr(r) + offset), pitch, ctypes.c_void_p(blk.ptr + offset),
                                         pitch, nbytes, rows, st)
            else:
                rc = L.jb_memcpy_async(ctypes.c_void_p(blk.peer_ptr(r) + offset), ctypes.c_void_p(blk.ptr + offset), nbytes, st)
            if rc == 0:
                rc = L.jb_memcpy_async(ctypes.c_void_p(blk.peer_ptr(r) + 4 * me), ctypes.c_void_p(word.data_ptr()), 4, st)
        done = torch.cuda.Event()
        done.record()
    if rc != 0:
        raise RuntimeError(f"jigsaw_b200: pushing a staged block to the peers failed with code {rc}")
    _lib.count_launches(1)
    return epoch, stride, replay, done



# --------------------------------------------------------------------------- neighbours
def neighbour_table(group_h: dist.ProcessGroup | None, group_w: dist.ProcessGroup | None) -> list[int | None]:
    """World rank of the tile at ``(sy, sx)`` relative to this rank for the 3x3 neighbourhood
    (index ``(sy + 1) * 3 + (sx + 1)``), ``None`` outside the tile grid.  Process meshes are
    regular grids, so a diagonal neighbour follows from the strides of the two axes."""

    def axis(g: dist.ProcessGroup | None) -> tuple[int, int, int]:
        if g is None or g.size() == 1:
            return 0, 1, 0
        ranks = dist.get_process_group_ranks(g)
        return g.rank(), g.size(), ranks[1] - ranks[0]

    rh, nh, sh = axis(group_h)
    rw, nw, sw = axis(group_w)
    me = dist.get_rank() if dist.is_initialized() else 0
    table: list[int | None] = []
    for sy in (-1, 0, 1):
        for sx in (-1, 0, 1):
            if (sy, sx) == (0, 0) or not (0 <= rh + sy < nh and 0 <= rw + sx < nw):
                table.append(None)
            else:
                table.append(me + sy * sh + sx * sw)
    return table


def make_halo(
    ar: PeerArena, nbrs: list[int | None], produce: Block | None, consume: Block | None
) -> "ctypes.pointer[JbHalo] | None":
    """Descriptor for one kernel launch: where to push the edges of ``produce`` (a new epoch is
    taken for it) and which flags to wait for before reading ``consume``."""
    if not ar.symmetric or all(n is None for n in nbrs):
        return None
    h = JbHalo()
    if produce is not None:
        h.push_epoch = ar.acquire(produce, nbrs)
        h.push_enabled = 1
        for d, n in enumerate(nbrs):
            if n is not None:
                h.push_buf[d] = produce.peer_ptr(n)
                h.push_flag[d] = ar.flag_ptr(n, produce.slot, 8 - d)
    if consume is not None and consume.slot >= 0:
        h.wait_epoch = consume.epoch
        h.wait_enabled = 1
        for d, n in enumerate(nbrs):
            if n is not None:
                h.wait_flag[d] = ar.flag_ptr(ar.rank, consume.slot, d)
    if ar._capture_stride is not None:
        h.replay = ar.replay.data_ptr()
        h.push_stride = h.wait_stride = ar._capture_stride
    return ctypes.pointer(h)
