"""Fused LayerNorm over a feature dimension split across GPUs (``csrc/norm.cu``).

Forward and backward are one kernel each: local row statistics, exchange of the per-row
partials with the other column ranks through peer memory (stores over NVLink + an epoch flag
per CTA), normalisation.  With an unsplit feature dimension the same kernels run without the
exchange.  Falls back (returns ``None``) for shapes / dtypes the kernels do not cover; the
caller then takes the ``torch.distributed`` path.

Reference parity: jigsaw/modules/normalization/_functional.py:45-59 (forward: two blocking
all-reduces) and :136-177 (backward: two more); here each direction is a single launch.
"""

from __future__ import annotations

import ctypes
from typing import Any

import torch
import torch.distributed as dist

from . import _lib, symm

_OK = (torch.float32, torch.bfloat16)


def _p(t: torch.Tensor | None) -> ctypes.c_void_p | None:
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"jigsaw_b200 kernel launcher {what} failed with code {rc}")


class _Exchange:
    """Inbox + flags of one launch.  With several column ranks they live in a symmetric arena
    block (same offset on every rank); the block goes back to the arena right after the launch
    is queued (reuse is ordered by the stream, the inbox halves alternate with the epoch)."""

    def __init__(self, device: torch.device, group: "dist.ProcessGroup | None | tuple", rows: int, grid: int, width: int = 2,
                 kind: str = "layer_norm") -> None:
        # ``group``: a process group, or ``(world ranks, my index)`` for the product of several groups
        if isinstance(group, tuple):
            peer_ranks, me = group
            parts = len(peer_ranks)
        else:
            parts = 1 if group is None else group.size()
            me = 0 if group is None else group.rank()
            peer_ranks = None if group is None else dist.get_process_group_ranks(group)
        self.desc = _lib.JbLnExchange()
        self.desc.parts, self.desc.me = parts, me
        self.block = None
        flag_bytes = (parts * grid * 4 + 255) // 256 * 256
        inbox_bytes = 2 * parts * rows * width * 4
        if parts == 1:
            self.local = torch.empty(inbox_bytes // 4, dtype=torch.float32, device=device)
            self.desc.inbox_local = self.local.data_ptr()
            return
        ar = symm.arena(device)
        self.block = ar.alloc(flag_bytes + inbox_bytes, tag=(kind, parts, rows, grid))
        self.desc.flag_local = self.block.ptr
        self.desc.inbox_local = self.block.ptr + flag_bytes
        for i, r in enumerate(peer_ranks):
            self.desc.flag_peer[i] = self.block.peer_ptr(r)
            self.desc.inbox_peer[i] = self.block.peer_ptr(r) + flag_bytes
        self.desc.epoch = ar.next_own_epoch(self.block)
        if ar.capture_stride is not None:
            self.desc.stride = ar.capture_stride
            self.desc.replay = ar.replay.data_ptr()
        self.arena = ar

    def done(self) -> None:
        if self.block is not None:
            self.arena.free(self.block)
            self.block = None


class _FusedLayerNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, x: torch.Tensor, w: torch.Tensor | None, b: torch.Tensor | None, group: Any, eps: float,
                out_dtype: torch.dtype) -> torch.Tensor:
        L = _lib.lib()
        dev = x.device
        n = x.shape[-1]
        x2 = x.reshape(-1, n)
        R = x2.shape[0]
        sm = _lib.sm_count(dev.index)
        grid = L.jb_layer_norm_grid2(R, n, 0, sm)
        y = torch.empty(x.shape, dtype=out_dtype, device=dev)
        mean = torch.empty(R, dtype=torch.float32, device=dev)
        rstd = torch.empty(R, dtype=torch.float32, device=dev)
        ex = _Exchange(dev, group, R, grid)
        status = symm.arena(dev).status
        _check(L.jb_layer_norm_fwd(_p(x2), int(x.dtype == torch.bfloat16), _p(y), int(out_dtype == torch.bfloat16), _p(w),
                                   _p(b), _p(mean), _p(rstd), R, n, float(eps), ctypes.byref(ex.desc), _p(status), sm,
                                   _lib.stream_ptr()), "layer_norm_fwd")
        ex.done()
        _lib.count_launches(1)
        ctx.save_for_backward(x2, w, mean, rstd)
        ctx.group, ctx.has_b, ctx.shape = group, b is not None, x.shape
        return y

    @staticmethod
    def backward(ctx: Any, g: torch.Tensor) -> tuple:
        L = _lib.lib()
        x2, w, mean, rstd = ctx.saved_tensors
        dev = x2.device
        R, n = x2.shape
        if g.dtype not in _OK:
            g = g.float()
        g2 = g.reshape(R, n).contiguous()
        sm = _lib.sm_count(dev.index)
        grid = L.jb_layer_norm_grid2(R, n, 1, sm)
        dx = torch.empty_like(x2)
        want_w = w is not None and ctx.needs_input_grad[1]
        want_b = ctx.has_b and ctx.needs_input_grad[2]
        dw = torch.empty(n, dtype=torch.float32, device=dev) if want_w else None
        db = torch.empty(n, dtype=torch.float32, device=dev) if want_b else None
        scratch = (torch.empty(L.jb_layer_norm_scratch_floats(R, n), dtype=torch.float32, device=dev)
                   if (want_w or want_b) else None)
        ex = _Exchange(dev, ctx.group, R, grid)
        status = symm.arena(dev).status
        _check(L.jb_layer_norm_bwd(_p(x2), int(x2.dtype == torch.bfloat16), _p(g2), int(g2.dtype == torch.bfloat16), _p(dx),
                                   int(dx.dtype == torch.bfloat16), _p(w), _p(mean), _p(rstd), _p(dw), _p(db), _p(scratch),
                                   R, n, ctypes.byref(ex.desc), _p(status), sm, _lib.stream_ptr()), "layer_norm_bwd")
        ex.done()
        _lib.count_launches(3 if scratch is not None else 1)
        return dx.view(ctx.shape), dw, db, None, None, None


@_lib.traced("jb.maybe_fused_layer_norm")
@_lib.audited("layer_norm")
def maybe_fused_layer_norm(x: torch.Tensor, w: torch.Tensor | None, b: torch.Tensor | None,
                           col_group: dist.ProcessGroup | None, eps: float) -> torch.Tensor | None:
    """LayerNorm of the last dimension of ``x`` (split over ``col_group``) with the fused
    kernels, or ``None`` when they do not apply."""
    if not x.is_cuda or x.dtype not in _OK or x.dim() < 2 or x.shape[-1] % 4 or x.shape[-1] > 12000 or x.numel() == 0:
        return None
    if any(t is not None and (t.dtype != torch.float32 or not t.is_contiguous()) for t in (w, b)):
        return None
    if b is not None and w is None:
        return None
    parts = 1 if col_group is None else col_group.size()
    if parts > 8 or torch._C._functorch.is_batchedtensor(x):
        return None
    if not _lib.available():
        raise RuntimeError("jigsaw_b200: the sm_100a kernel library is missing on a CUDA machine")
    out_dtype = torch.float32 if torch.is_autocast_enabled("cuda") else x.dtype
    return _FusedLayerNorm.apply(x.contiguous(), w, b, col_group if parts > 1 else None, eps, out_dtype)


# ----------------------------------------------------------------------------- GroupNorm
def _tile_ranks(groups: list) -> tuple[list[int], int]:
    """World ranks of every tile of the grid spanned by ``groups`` (regular mesh: the offsets
    along the axes add up) and this rank's index among them."""
    me = dist.get_rank()
    ranks = [me]
    for g in groups:
        gr = dist.get_process_group_ranks(g)
        mine = gr[g.rank()]
        ranks = [r + (o - mine) for r in ranks for o in gr]
    ranks = sorted(ranks)
    return ranks, ranks.index(me)


_gn_scratch: dict[int, torch.Tensor] = {}


class _FusedGroupNorm(torch.autograd.Function):
    """GroupNorm of ``x [N, C, *spatial]`` whose spatial extent is tiled over ``groups``: one launch
    per direction (chunk statistics, grid barrier, in-kernel exchange between the tile ranks,
    normalisation)."""

    @staticmethod
    def forward(ctx: Any, x: torch.Tensor, w: torch.Tensor | None, b: torch.Tensor | None, groups_local: int, tiles: Any,
                eps: float, out_dtype: torch.dtype) -> torch.Tensor:
        L, dev = _lib.lib(), x.device
        N, C = x.shape[0], x.shape[1]
        S = x.numel() // (N * C)
        cg = C // groups_local
        G = N * groups_local
        sm = _lib.sm_count(dev.index)
        splits = L.jb_group_norm_splits(G, sm)
        y = torch.empty(x.shape, dtype=out_dtype, device=dev)
        stats = torch.empty(G, 2, dtype=torch.float32, device=dev)
        partial = torch.empty(G * splits, 4, dtype=torch.float32, device=dev)
        if dev.index not in _gn_scratch:
            _gn_scratch[dev.index] = torch.zeros(4, dtype=torch.int32, device=dev)
        counters = _gn_scratch[dev.index]
        ex = _Exchange(dev, tiles, G, G, width=4, kind="group_norm")
        status = symm.arena(dev).status
        _check(L.jb_group_norm_fwd(_p(x), int(x.dtype == torch.bfloat16), _p(y), int(out_dtype == torch.bfloat16), _p(w), _p(b),
                                   _p(stats), _p(partial), _p(counters), G, groups_local, cg, S, float(eps),
                                   ctypes.byref(ex.desc), _p(status), sm, _lib.stream_ptr()), "group_norm_fwd")
        ex.done()
        _lib.count_launches(1)
        ctx.save_for_backward(x, w, stats)
        ctx.meta = (groups_local, tiles, b is not None)
        return y

    @staticmethod
    def backward(ctx: Any, g: torch.Tensor) -> tuple:
        L = _lib.lib()
        x, w, stats = ctx.saved_tensors
        groups_local, tiles, has_b = ctx.meta
        dev = x.device
        N, C = x.shape[0], x.shape[1]
        S = x.numel() // (N * C)
        cg = C // groups_local
        G = N * groups_local
        sm = _lib.sm_count(dev.index)
        splits = L.jb_group_norm_splits(G, sm)
        if g.dtype not in _OK:
            g = g.float()
        g = g.contiguous()
        dx = torch.empty_like(x)
        partial = torch.empty(G * splits, 4, dtype=torch.float32, device=dev)
        dwp = torch.empty(N, groups_local, splits, cg, dtype=torch.float32, device=dev)
        dbp = torch.empty(N, groups_local, splits, cg, dtype=torch.float32, device=dev)
        counters = _gn_scratch[dev.index]
        ex = _Exchange(dev, tiles, G, G, width=4, kind="group_norm")
        status = symm.arena(dev).status
        _check(L.jb_group_norm_bwd(_p(x), int(x.dtype == torch.bfloat16), _p(g), int(g.dtype == torch.bfloat16), _p(dx),
                                   int(dx.dtype == torch.bfloat16), _p(w), _p(stats), _p(partial), _p(dwp), _p(dbp),
                                   _p(counters), G, groups_local, cg, S, ctypes.byref(ex.desc), _p(status), sm,
                                   _lib.stream_ptr()), "group_norm_bwd")
        ex.done()
        _lib.count_launches(1)
        dw = dwp.sum(dim=(0, 2)).reshape(C) if (w is not None and ctx.needs_input_grad[1]) else None
        db = dbp.sum(dim=(0, 2)).reshape(C) if (has_b and ctx.needs_input_grad[2]) else None
        return dx, dw, db, None, None, None, None


@_lib.traced("jb.maybe_fused_group_norm")
@_lib.audited("group_norm")
def maybe_fused_group_norm(x: torch.Tensor, groups_local: int, w: torch.Tensor | None, b: torch.Tensor | None,
                           spatial_groups: list, eps: float) -> torch.Tensor | None:
    """GroupNorm with statistics over the tiles of ``spatial_groups`` on the fused kernels, or
    ``None`` when they do not apply."""
    if not x.is_cuda or x.dtype not in _OK or x.dim() < 3 or x.numel() == 0 or x.numel() >= 2 ** 40:
        return None
    N, C = x.shape[0], x.shape[1]
    S = x.numel() // (N * C)
    if C % groups_local or S % 4 or C // groups_local > 256 or torch._C._functorch.is_batchedtensor(x):
        return None
    if any(t is not None and (t.dtype != torch.float32 or not t.is_contiguous()) for t in (w, b)) or (b is not None and w is None):
        return None
    live = [g for g in spatial_groups if g is not None and g.size() > 1]
    tiles = _tile_ranks(live) if live else None
    if tiles is not None and len(tiles[0]) > 8:
        return None
    if not _lib.available():
        raise RuntimeError("jigsaw_b200: the sm_100a kernel library is missing on a CUDA machine")
    if _lib.lib().jb_group_norm_splits(N * groups_local, _lib.sm_count(x.device.index)) <= 0:
        return None
    out_dtype = torch.float32 if torch.is_autocast_enabled("cuda") else x.dtype
    return _FusedGroupNorm.apply(x.contiguous(), w, b, groups_local, tiles, eps, out_dtype)
