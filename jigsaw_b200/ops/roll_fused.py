"""Fused distributed roll (``csrc/roll.cu``): one kernel stores every element at its destination,
in this GPU's output or directly in a neighbour's over NVLink, publishes an epoch flag and waits
for the neighbours' flags; no slab is cut, sent or concatenated.  Handles one or two rolled
dimensions, each tiled over a group or local, and any shift.

Reference parity: ``torch.roll`` + slab exchange + overwrite in
jigsaw/modules/roll/_distributed_roll.py:44-59,99 (one blocking exchange per distributed
dimension there).
"""

from __future__ import annotations

import ctypes
from typing import Any

import torch
import torch.distributed as dist

from . import _lib, symm

_HEADER = 256


def _ring_block(ar: "symm.PeerArena", tag: tuple, nbytes: int) -> "symm.Block":
    """The next block of the two-deep staging ring ``tag`` (:meth:`symm.PeerArena.ring_block`)."""
    return ar.ring_block(tag, nbytes)


def _axis(group: Any, shift: int, n: int) -> tuple[int, int, list[int], int]:
    """(remainder, ranks of the two destinations as world ranks, two sources, ...) helper:
    returns ``(rem, [dest0, dest1], [src0, src1], G)`` in group-rank terms."""
    G = 1 if group is None else group.size()
    r = 0 if group is None else group.rank()
    s = shift % (G * n)
    q, rem = divmod(s, n)
    dests = [(r + q) % G, (r + q + 1) % G]
    srcs = [(r - q) % G, (r - q - 1) % G]
    return rem, dests, srcs, G


class _FusedRoll(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, x: torch.Tensor, shifts: tuple, dims: tuple, groups: tuple) -> torch.Tensor:
        ctx.shifts, ctx.dims, ctx.groups = shifts, dims, groups
        return _launch(x, shifts, dims, groups)

    @staticmethod
    def backward(ctx: Any, g: torch.Tensor) -> tuple:
        return _launch(g.contiguous(), tuple(-s for s in ctx.shifts), ctx.dims, ctx.groups), None, None, None


def _launch(x: torch.Tensor, shifts: tuple, dims: tuple, groups: tuple) -> torch.Tensor:
    L, dev = _lib.lib(), x.device
    ar = symm.arena(dev)
    shape = x.shape
    d1 = dims[0]
    two = len(dims) == 2
    d2 = dims[1] if two else d1
    A = 1
    for n in shape[:d1]:
        A *= n
    H = shape[d1]
    M = 1
    for n in shape[d1 + 1:d2]:
        M *= n
    W = shape[d2] if two else 1
    tail = 1
    for n in shape[d2 + 1:]:
        tail *= n
    I16 = tail * x.element_size() // 16
    gh, gw = groups[0], (groups[1] if two else None)
    rem_h, dest_h, src_h, Gh = _axis(gh, shifts[0], H)
    rem_w, dest_w, src_w, Gw = _axis(gw, shifts[1], W) if two else (0, [0, 0], [0, 0], 1)
    ranks_h = [dist.get_rank()] if gh is None else dist.get_process_group_ranks(gh)
    ranks_w = [dist.get_rank()] if gw is None else dist.get_process_group_ranks(gw)
    me = dist.get_rank()
    rh = 0 if gh is None else gh.rank()
    rw = 0 if gw is None else gw.rank()

    def world(ih: int, iw: int) -> int:        # regular tile grid: offsets along the two axes add up
        return me + (ranks_h[ih] - ranks_h[rh]) + (ranks_w[iw] - ranks_w[rw])

    nbytes = x.numel() * x.element_size()
    blk = _ring_block(ar, ("roll", dev.index, nbytes, tuple(ranks_h), tuple(ranks_w)), _HEADER + nbytes)
    epoch = ar.next_own_epoch(blk)
    r = _lib.JbRoll()
    r.x, r.A, r.M, r.I16, r.H, r.W, r.rem_h, r.rem_w = x.data_ptr(), A, M, I16, H, W, rem_h, rem_w
    for ah in (0, 1):
        for aw in (0, 1):
            k = ah * 2 + aw
            dst = world(dest_h[ah], dest_w[aw])
            src = world(src_h[ah], src_w[aw])
            r.out[k] = (blk.ptr if dst == me else blk.peer_ptr(dst)) + _HEADER
            r.flag_out[k] = None if dst == me else blk.peer_ptr(dst) + 4 * k
            r.flag_in[k] = None if src == me else blk.ptr + 4 * k
    r.epoch = epoch
    if ar.capture_stride is not None:
        r.stride, r.replay = ar.capture_stride, ar.replay.data_ptr()
    rc = L.jb_roll(ctypes.byref(r), ctypes.c_void_p(ar.done_counter.data_ptr()), ctypes.c_void_p(ar.status.data_ptr()),
                   _lib.sm_count(dev.index), _lib.stream_ptr())
    if rc != 0:
        raise RuntimeError(f"jigsaw_b200 kernel launcher roll failed with code {rc}")
    _lib.count_launches(1)
    return blk.tensor[_HEADER:_HEADER + nbytes].view(x.dtype).view(shape).clone()


@_lib.traced("jb.maybe_fused_roll")
@_lib.audited("roll")
def maybe_fused_roll(x: torch.Tensor, shifts: tuple, dims: tuple, where: dict) -> torch.Tensor | None:
    """Roll ``x`` by ``shifts`` along ``dims``; ``where`` maps a dimension to the group that tiles
    it.  ``None`` when the kernel does not apply."""
    nd = x.dim()
    dims = tuple(d % nd for d in dims)
    if not x.is_cuda or len(dims) not in (1, 2) or len(set(dims)) != len(dims) or x.numel() == 0:
        return None
    if not any(where.get(d) is not None and where[d].size() > 1 for d in dims) or not dist.is_initialized():
        return None                                  # nothing is tiled: torch.roll is already one kernel
    order = sorted(range(len(dims)), key=lambda i: dims[i])
    dims = tuple(dims[i] for i in order)
    shifts = tuple(int(shifts[i]) for i in order)
    groups = tuple(where.get(d) if where.get(d) is not None and where[d].size() > 1 else None for d in dims)
    tail = 1
    for n in x.shape[dims[-1] + 1:]:
        tail *= n
    if (tail * x.element_size()) % 16 or torch._C._functorch.is_batchedtensor(x):
        return None
    if not _lib.available():
        raise RuntimeError("jigsaw_b200: the sm_100a kernel library is missing on a CUDA machine")
    return _FusedRoll.apply(x.contiguous(), shifts, dims, groups)
