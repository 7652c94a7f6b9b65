"""Ulysses attention: both exchanges fused into the projections next to them (opt-in, see the switches below).

QKV projection (sequence -> head exchange in the epilogue):

The projection ``x @ W_qkv.T`` of a sequence shard produces, for every head group ``p``, the
columns that rank ``p`` needs.  With the rows of ``W_qkv`` ordered (head group, q|k|v, head, d)
those columns are one contiguous part, and the scatter epilogue of the tcgen05 GEMM
(``csrc/gemm.cu``) stores each output tile straight into rank ``p``'s inbox as it is produced: the
all-to-all rides inside the GEMM, tile by tile, and the projected ``(b, s / P, 3 h d)`` tensor is
never written locally.  The receiver waits for the senders' flags and views its inbox as
``(3, b, s, h / P, d)``.  The backward pass sends the gradient back with the peer-memory
all-to-all kernel and runs the two remaining products on the same GEMM kernel.

Output projection (head -> sequence exchange in the operand loads): every rank stages its heads ordered
by destination; the GEMM of rank ``r`` loads k-block part ``p`` (the heads of rank ``p``) by TMA from
rank ``p``'s staging block, so the exchanged tensor is never materialised.  Its input gradient is again
a scatter-epilogue GEMM.

Both forms give the results of the unfused path on 2 GPUs; neither measured faster there (the
epilogue's 64-byte row stores use NVLink poorly), so the attention layer uses them only when the
switches ``FUSE_QKV_PROJECTION`` / ``FUSE_OUTPUT_PROJECTION`` are set.

Reference parity: the projection followed by ``all_to_all_single`` in
jigsaw/modules/attention/_functional/ulysses.py:19-63.
"""

from __future__ import annotations

import ctypes
import os
from typing import Any

import torch
import torch.distributed as dist

from . import _lib, symm
from .linear_fused import _HEADER, _staging_block, gemm, scatter_gemm_launcher


def head_group_major(w: torch.Tensor, parts: int, heads: int, head_dim: int) -> torch.Tensor:
    """Rows of a qkv weight ``(3 h d, in)`` reordered from (q|k|v, head, d) to
    (head group, q|k|v, head in group, d)."""
    k = w.shape[1]
    return w.view(3, parts, heads // parts, head_dim, k).permute(1, 0, 2, 3, 4).reshape(3 * heads * head_dim, k)


def inbox_to_qkv(inbox: torch.Tensor, parts: int, b: int, sl: int, hl: int, d: int) -> torch.Tensor:
    """``inbox`` holds one slab per source rank, each ``(b * sl, 3 * hl * d)``; returns the gathered
    ``(3, b, parts * sl, hl, d)`` (source rank ``r`` owns sequence block ``r``)."""
    t = inbox.view(parts, b, sl, 3, hl, d).permute(3, 1, 0, 2, 4, 5)
    return t.reshape(3, b, parts * sl, hl, d)


def from_head_group_major(wp: torch.Tensor, parts: int, heads: int, head_dim: int) -> torch.Tensor:
    """Inverse of :func:`head_group_major` (used for the weight gradient)."""
    k = wp.shape[1]
    return wp.view(parts, 3, heads // parts, head_dim, k).permute(1, 0, 2, 3, 4).reshape(3 * heads * head_dim, k)


def grad_columns(back: torch.Tensor, parts: int, b: int, sl: int, hl: int, d: int) -> torch.Tensor:
    """Gradient of the local projection ``(3, b, sl, h, d)`` as a matrix ``(b * sl, 3 h d)`` whose
    columns follow the row order of :func:`head_group_major`."""
    return back.view(3, b, sl, parts, hl, d).permute(1, 2, 3, 0, 4, 5).reshape(b * sl, 3 * parts * hl * d)


def _scatter_exchange(a: torch.Tensor, bmat: torch.Tensor, b_mn: bool, cols: int, group: Any, tag: str) -> torch.Tensor:
    """``a @ B`` (``a`` is ``[M, K]``; ``bmat`` is ``[P * cols, K]``, or ``[K, P * cols]`` with ``b_mn``)
    whose column part ``p`` is stored by the GEMM epilogue into rank ``p``'s inbox; returns this
    rank's inbox ``(P, M, cols)`` (slab ``r`` written by rank ``r``) once every sender's flag has
    arrived.  The inbox is a view of a block that is reused two calls later: copy out of it."""
    L, dev = _lib.lib(), a.device
    ar = symm.arena(dev)
    P, me = group.size(), group.rank()
    ranks = dist.get_process_group_ranks(group)
    M, K = a.shape
    slab = M * cols * 2
    blk = _staging_block(ar, (tag, dev.index, M, cols, tuple(ranks)), _HEADER + P * slab)
    epoch = ar.next_own_epoch(blk)
    stride = ar.capture_stride or 0
    replay = ar.replay.data_ptr() if ar.capture_stride is not None else None
    st = _lib.stream_ptr()
    status = ctypes.c_void_p(ar.status.data_ptr())
    c_part = (ctypes.c_void_p * 8)()
    for i, r in enumerate(ranks):
        c_part[i] = (blk.ptr if i == me else blk.peer_ptr(r)) + _HEADER + me * slab
    rc = scatter_gemm_launcher(L)(ctypes.c_void_p(a.data_ptr()), ctypes.c_void_p(bmat.data_ptr()), c_part, P, cols, M, K,
                                a.stride(0), bmat.stride(0), 0, 1 if b_mn else 0, _lib.sm_count(dev.index), status, st)
    flags = (ctypes.c_void_p * 8)()
    waits = (ctypes.c_void_p * 8)()
    n = 0
    for i, r in enumerate(ranks):
        if i != me:
            flags[n] = blk.peer_ptr(r) + 4 * me
            waits[n] = blk.ptr + 4 * i
            n += 1
    if rc == 0:
        rc = L.jb_publish(flags, n, epoch, stride, replay, st)
    if rc == 0:
        rc = L.jb_wait_flags(waits, n, epoch, stride, replay, status, st)
    if rc != 0:
        raise RuntimeError(f"jigsaw_b200 kernel launcher {tag} failed with code {rc}")
    _lib.count_launches(3)
    return blk.tensor[_HEADER:_HEADER + P * slab].view(torch.bfloat16).view(P, M, cols)


def _bf16(t: torch.Tensor) -> torch.Tensor:
    return t if t.dtype == torch.bfloat16 else t.to(torch.bfloat16)


class _UlyssesQKV(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, x: torch.Tensor, w: torch.Tensor, group: Any, heads: int, head_dim: int) -> torch.Tensor:
        P = group.size()
        b, sl, K = x.shape
        hl = heads // P
        xb = _bf16(x.reshape(b * sl, K))
        xb = xb if xb.is_contiguous() else xb.contiguous()
        wp = head_group_major(_bf16(w), P, heads, head_dim).contiguous()
        inbox = _scatter_exchange(xb, wp, False, 3 * hl * head_dim, group, "ulysses_qkv")
        out = inbox_to_qkv(inbox, P, b, sl, hl, head_dim).contiguous()
        ctx.save_for_backward(xb, wp)
        ctx.meta = (group, heads, head_dim, x.shape, x.dtype, w.dtype)
        return out

    @staticmethod
    def backward(ctx: Any, g: torch.Tensor) -> tuple:
        from .._core.collectives import all_to_all_dims

        xb, wp = ctx.saved_tensors
        group, heads, d, x_shape, x_dtype, w_dtype = ctx.meta
        P = group.size()
        b, sl = x_shape[0], x_shape[1]
        g = g if g.dtype == torch.bfloat16 else g.to(torch.bfloat16)
        # (3, b, s, h / P, d) -> (3, b, s / P, h, d): the inverse exchange (one peer-memory kernel)
        back = all_to_all_dims(g.contiguous(), group, split_dim=-3, cat_dim=-2)
        hl = heads // P
        g2 = grad_columns(back, P, b, sl, hl, d).contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = gemm(g2, wp, b_mn=True).view(x_shape).to(x_dtype)
        if ctx.needs_input_grad[1]:
            dwp = gemm(g2, xb, a_mn=True, b_mn=True, out_dtype=torch.float32)          # rows ordered like wp
            dw = from_head_group_major(dwp, P, heads, d).to(w_dtype)
        return dx, dw, None, None, None


# Switches of the two fused projections.  The QKV projection with the exchange in its epilogue is off by
# default: on 2 GPUs it measured 0.55 ms against 0.41 ms for the GEMM followed by the all-to-all kernel
# (batch 8, 4096 tokens, width 1024), because the epilogue's 64-byte row stores use NVLink poorly.
FUSE_QKV_PROJECTION = os.environ.get("JIGSAW_FUSE_ULYSSES_QKV", "0") == "1"
FUSE_OUTPUT_PROJECTION = os.environ.get("JIGSAW_FUSE_ULYSSES_OUT", "0") == "1"


def stage_for_owners(o: torch.Tensor, parts: int) -> torch.Tensor:
    """``o`` is this rank's attention output ``(b, s, hl, d)`` (heads of this rank, whole sequence);
    returns the view ``(parts, b, s / parts, hl, d)`` whose entry ``r`` is what rank ``r`` needs."""
    return o.unflatten(1, (parts, o.shape[1] // parts)).permute(1, 0, 2, 3, 4)


class _UlyssesOut(torch.autograd.Function):
    """Output projection of Ulysses attention with the head -> sequence exchange as the gather of its
    A operand: every rank stages its heads ordered by destination, and the GEMM of rank ``r`` loads
    k-block part ``p`` (the heads of rank ``p``) by TMA from rank ``p``'s staging block."""

    @staticmethod
    def forward(ctx: Any, o: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, group: Any) -> torch.Tensor:
        L, dev = _lib.lib(), o.device
        ar = symm.arena(dev)
        P, me = group.size(), group.rank()
        ranks = dist.get_process_group_ranks(group)
        b, s, hl, d = o.shape
        sl, kp = s // P, hl * d
        M, N = b * sl, w.shape[0]
        part = M * kp * 2
        blk = _staging_block(ar, ("ulysses_out", dev.index, M, kp, tuple(ranks)), _HEADER + P * part)
        staged = blk.tensor[_HEADER:_HEADER + P * part].view(torch.bfloat16).view(P, b, sl, hl, d)
        staged.copy_(stage_for_owners(o, P))                               # cast + reorder in one kernel
        epoch = ar.next_own_epoch(blk)
        stride = ar.capture_stride or 0
        replay = ar.replay.data_ptr() if ar.capture_stride is not None else None
        st = _lib.stream_ptr()
        flags = (ctypes.c_void_p * 8)()
        n = 0
        for i, r in enumerate(ranks):
            if i != me:
                flags[n] = blk.peer_ptr(r) + 4 * me
                n += 1
        rc = L.jb_publish(flags, n, epoch, stride, replay, st)
        g = _lib.JbGather()
        for i, r in enumerate(ranks):
            g.a_part[i] = (blk.ptr if i == me else blk.peer_ptr(r)) + _HEADER + me * part
            g.flag[i] = None if i == me else blk.ptr + 4 * i
        g.epoch, g.stride, g.replay, g.parts, g.k_part, g.lda_part = epoch, stride, replay, P, kp, kp
        wb = _bf16(w)
        wb = wb if wb.is_contiguous() else wb.contiguous()
        fb = None if bias is None else bias.float().contiguous()
        y = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        if rc == 0:
            rc = L.jb_gemm_bf16_gather(ctypes.byref(g), ctypes.c_void_p(wb.data_ptr()), ctypes.c_void_p(y.data_ptr()),
                                       None if fb is None else ctypes.c_void_p(fb.data_ptr()), M, N, wb.stride(0),
                                       y.stride(0), 0, 0, _lib.sm_count(dev.index), ctypes.c_void_p(ar.status.data_ptr()), st)
        if rc != 0:
            raise RuntimeError(f"jigsaw_b200 kernel launcher ulysses_out failed with code {rc}")
        _lib.count_launches(2)
        ctx.save_for_backward(o if ctx.needs_input_grad[1] else None, wb)
        ctx.meta = (group, o.shape, o.dtype, w.dtype, None if bias is None else bias.dtype)
        return y.view(b, sl, N)

    @staticmethod
    def backward(ctx: Any, gy: torch.Tensor) -> tuple:
        from .._core.collectives import all_to_all_dims

        o, wb = ctx.saved_tensors
        group, o_shape, o_dtype, w_dtype, b_dtype = ctx.meta
        P = group.size()
        b, s, hl, d = o_shape
        sl, kp, N = s // P, hl * d, wb.shape[0]
        g = _bf16(gy.reshape(b * sl, N))
        g = g if g.is_contiguous() else g.contiguous()
        do = dw = db = None
        if ctx.needs_input_grad[0]:
            # g @ W is the gradient of the gathered heads; column part p belongs to rank p (scatter epilogue)
            inbox = _scatter_exchange(g, wb, True, kp, group, "ulysses_out_grad")
            do = inbox.view(P, b, sl, hl, d).permute(1, 0, 2, 3, 4).reshape(b, s, hl, d).to(o_dtype)
        if ctx.needs_input_grad[1]:
            mine = all_to_all_dims(_bf16(o).contiguous(), group, split_dim=-3, cat_dim=-2)     # (b, sl, h, d)
            dw = gemm(g, mine.view(b * sl, P * kp), a_mn=True, b_mn=True, out_dtype=torch.float32).to(w_dtype)
        if b_dtype is not None and ctx.needs_input_grad[2]:
            db = g.sum(dim=0, dtype=torch.float32).to(b_dtype)
        return do, dw, db, None


@_lib.traced("jb.maybe_fused_ulysses_out")
def maybe_fused_ulysses_out(o: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, group: Any) -> torch.Tensor | None:
    """``heads_to_seq(o).flatten(-2) @ w.T + bias`` as ``(b, s / P, N)`` in bf16 with the exchange fused
    into the GEMM's operand loads, or ``None`` when that does not apply.  ``o`` is ``(b, s, heads / P,
    head_dim)``, ``w`` is ``(N, heads * head_dim)``."""
    if not FUSE_OUTPUT_PROJECTION or group is None or not o.is_cuda or o.dim() != 4 or w.dim() != 2 or o.numel() == 0:
        return None
    P = group.size()
    bf16 = o.dtype == torch.bfloat16 or (torch.is_autocast_enabled("cuda") and torch.get_autocast_dtype("cuda") == torch.bfloat16)
    if not bf16 or P < 2 or P > 8 or o.shape[1] % P:
        return None
    b, s, hl, d = o.shape
    kp, N, M = hl * d, w.shape[0], b * (s // P)
    if w.shape[1] != P * kp or kp % 64 or N % 8 or N < 16 or M % 8 or torch._C._functorch.is_batchedtensor(o):
        return None
    if o.dtype not in (torch.float32, torch.bfloat16, torch.float16) or w.dtype not in (torch.float32, torch.bfloat16):
        return None
    if bias is not None and bias.dtype not in (torch.float32, torch.bfloat16):
        return None
    if not _lib.available():
        raise RuntimeError("jigsaw_b200: the sm_100a kernel library is missing on a CUDA machine")
    return _UlyssesOut.apply(o, w, bias, group)


@_lib.traced("jb.maybe_fused_ulysses_qkv")
def maybe_fused_ulysses_qkv(x: torch.Tensor, w: torch.Tensor, group: Any, heads: int, head_dim: int) -> torch.Tensor | None:
    """``seq_to_heads(split_heads(x @ w.T))`` as ``(3, b, s, heads / P, head_dim)`` in bf16 with the
    exchange fused into the GEMM epilogue, or ``None`` when that does not apply.  ``x`` is
    ``(b, s / P, in)``, ``w`` is ``(3 * heads * head_dim, in)``."""
    if not FUSE_QKV_PROJECTION or group is None or not x.is_cuda or x.dim() != 3 or w.dim() != 2 or x.numel() == 0:
        return None
    P = group.size()
    bf16 = x.dtype == torch.bfloat16 or (torch.is_autocast_enabled("cuda") and torch.get_autocast_dtype("cuda") == torch.bfloat16)
    if not bf16 or P < 2 or P > 8 or heads % P or w.shape[0] != 3 * heads * head_dim:
        return None
    K = x.shape[-1]
    cols = 3 * (heads // P) * head_dim
    M = x.shape[0] * x.shape[1]
    if K % 64 or cols % 64 or M % 8 or torch._C._functorch.is_batchedtensor(x):
        return None
    if x.dtype not in (torch.float32, torch.bfloat16) or w.dtype not in (torch.float32, torch.bfloat16):
        return None
    if not _lib.available():
        raise RuntimeError("jigsaw_b200: the sm_100a kernel library is missing on a CUDA machine")
    return _UlyssesQKV.apply(x, w, group, heads, head_dim)
