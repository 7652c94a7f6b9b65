"""Attention on the GPU.

* :class:`FlashAttention` / :func:`flash_attention_forward` / :func:`flash_attention_backward`: attention
  for head dimension 64 on the tcgen05 kernels of ``csrc/flash_attn.cu`` and ``csrc/flash_attn_bwd.cu``.
* :func:`maybe_fused_ring_attention`: sequence-parallel (ring) attention as ONE forward launch and two
  backward launches.  Every rank pushes its keys / values (backward: also queries, output gradients,
  log-sum-exp and D) into its slot of every peer's staging block with the copy engines, followed by a flag,
  so each part crosses NVLink once per destination and no SM moves data; the kernels start on their own part
  at once, walk over the parts of all ranks as their flags arrive (bounded waits) and load every block by TMA
  from local memory while the previous block is in the tensor cores.  The running softmax state stays on chip
  across the parts, so there is no per-chunk merge, and every rank computes the complete gradient of its own
  keys and values from the other ranks' queries, so no gradient travels back.
* :func:`maybe_fused_merge`: the online-softmax merge of per-chunk results (``csrc/elementwise.cu``), used
  by the chunked ring schedule that remains for what the fused kernels do not cover (other head sizes,
  dropout, circulating ``x``, CPU).

Reference parity: jigsaw/modules/attention/_functional/forward.py:102-200 and backward.py:109-312 (ring
drivers), cores/sdpa.py:17-165 (per-chunk core), _merge_kernel.py:37-82 (merge).
"""

from __future__ import annotations

import ctypes
from typing import Any

import torch
import torch.distributed as dist

from . import _lib, symm


@_lib.traced("jb.maybe_fused_merge")
@_lib.audited("merge")
def maybe_fused_merge(out: torch.Tensor, lse: torch.Tensor, out_j: torch.Tensor, lse_j: torch.Tensor):
    """In place: ``out += sigmoid(lse_j - lse) (out_j - out)``, ``lse = logaddexp(lse, lse_j)``;
    returns ``(out, lse)``, or ``None`` when the kernel does not apply (the state must be
    contiguous fp32 and must not be tracked by autograd)."""
    if (out.dtype != torch.float32 or lse.dtype != torch.float32 or out_j.dtype not in (torch.float32, torch.bfloat16)
            or out.requires_grad or out_j.requires_grad or lse.requires_grad or lse_j.requires_grad):
        return None
    if not (out.is_contiguous() and lse.is_contiguous() and out_j.is_contiguous()) or out.shape != out_j.shape:
        return None
    if lse.shape != out.shape[:-1] or lse_j.shape != lse.shape or out.numel() == 0:
        return None
    if torch._C._functorch.is_batchedtensor(out) or not _lib.available():
        return None
    lj = lse_j.float().contiguous()
    d = out.shape[-1]
    rc = _lib.lib().jb_merge_chunks(ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(lse.data_ptr()),
                                    ctypes.c_void_p(out_j.data_ptr()), int(out_j.dtype == torch.bfloat16),
                                    ctypes.c_void_p(lj.data_ptr()), out.numel() // d, d, _lib.stream_ptr())
    if rc != 0:
        raise RuntimeError(f"jigsaw_b200 kernel launcher merge_chunks failed with code {rc}")
    _lib.count_launches(1)
    return out, lse


@_lib.traced("jb.flash_attention_forward")
def flash_attention_forward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float) -> tuple[torch.Tensor, torch.Tensor]:
    """``softmax(scale * q k^T) v`` and the row-wise log-sum-exp on the tcgen05 kernel of
    ``csrc/flash_attn.cu``.  ``q`` is ``(..., sq, 64)``, ``k`` and ``v`` are ``(..., sk, 64)``, all bf16 on
    one CUDA device with equal leading dimensions; returns ``(out bf16 (..., sq, 64), lse fp32 (..., sq))``.
    Forward only (no autograd): :class:`FlashAttention` is the differentiable form.

    Reference parity: the role of the SDPA flash core, jigsaw/modules/attention/_functional/cores/sdpa.py:17-165.
    """
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16:
        raise TypeError("flash_attention_forward needs bf16 inputs")
    if q.shape[-1] != 64 or k.shape[-1] != 64 or v.shape[-1] != 64 or k.shape != v.shape or q.shape[:-2] != k.shape[:-2]:
        raise ValueError("flash_attention_forward needs head dimension 64 and matching leading dimensions")
    if not _lib.available():
        raise RuntimeError("jigsaw_b200: the sm_100a kernel library is missing on a CUDA machine")
    lead = q.shape[:-2]
    sq, sk = q.shape[-2], k.shape[-2]
    q3, k3, v3 = (t.reshape(-1, t.shape[-2], 64).contiguous() for t in (q, k, v))
    bh = q3.shape[0]
    out = torch.empty_like(q3)
    lse = torch.empty(bh, sq, dtype=torch.float32, device=q.device)
    status = None
    if bh > 0 and sq > 0:
        ar = symm.arena(q.device)
        status = ar.status
        rc = _lib.lib().jb_flash_attn_fwd(
            ctypes.c_void_p(q3.data_ptr()), ctypes.c_void_p(k3.data_ptr()), ctypes.c_void_p(v3.data_ptr()),
            ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(lse.data_ptr()), bh, sq, sk,
            q3.stride(1), q3.stride(0), k3.stride(1), k3.stride(0), v3.stride(1), v3.stride(0), out.stride(1), out.stride(0),
            float(scale), ctypes.c_void_p(status.data_ptr()), _lib.stream_ptr())
        if rc != 0:
            raise RuntimeError(f"jigsaw_b200 kernel launcher flash_attn_fwd failed with code {rc}")
        _lib.count_launches(1)
    return out.view(*lead, sq, 64), lse.view(*lead, sq)


@_lib.traced("jb.flash_attention_backward")
def flash_attention_backward(dout: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor,
                             lse: torch.Tensor, scale: float) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Gradients of :func:`flash_attention_forward` (``csrc/flash_attn_bwd.cu``): ``lse`` is the forward's
    log-sum-exp, ``out`` its output; returns ``(dq, dk, dv)`` in bf16 with the shapes of ``q``, ``k``, ``v``."""
    from . import symm

    sq, sk = q.shape[-2], k.shape[-2]
    q3, k3, v3, o3, g3 = (t.to(torch.bfloat16).reshape(-1, t.shape[-2], 64).contiguous() for t in (q, k, v, out, dout))
    bh = q3.shape[0]
    lse2 = lse.float().reshape(bh, sq).contiguous()
    delta = torch.empty_like(lse2)
    dq, dk, dv = torch.empty_like(q3), torch.empty_like(k3), torch.empty_like(v3)
    P = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    rc = _lib.lib().jb_flash_attn_bwd(P(q3), P(k3), P(v3), P(o3), P(g3), P(lse2), P(delta), P(dq), P(dk), P(dv),
                                      bh, sq, sk, float(scale), P(symm.arena(q.device).status), _lib.stream_ptr())
    if rc != 0:
        raise RuntimeError(f"jigsaw_b200 kernel launcher flash_attn_bwd failed with code {rc}")
    _lib.count_launches(3)
    return dq.view(q.shape), dk.view(k.shape), dv.view(v.shape)


class FlashAttention(torch.autograd.Function):
    """``softmax(scale * q k^T) v`` with forward and backward on the tcgen05 kernels
    (``csrc/flash_attn.cu``, ``csrc/flash_attn_bwd.cu``); same shapes as :func:`flash_attention_forward`."""

    @staticmethod
    def forward(ctx, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float) -> torch.Tensor:
        out, lse = flash_attention_forward(q, k, v, scale)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.scale = float(scale)
        return out

    @staticmethod
    def backward(ctx, g: torch.Tensor) -> tuple:
        q, k, v, out, lse = ctx.saved_tensors
        return (*flash_attention_backward(g, q, k, v, out, lse, ctx.scale), None)


def flash_usable(q: torch.Tensor, k: torch.Tensor, dropout_p: float = 0.0) -> bool:
    """Whether the tcgen05 attention kernels cover these operands."""
    return (q.is_cuda and q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16 and q.shape[-1] == 64 and k.shape[-1] == 64
            and dropout_p == 0.0 and q.shape[:-2] == k.shape[:-2] and q.numel() > 0 and k.numel() > 0
            and not torch._C._functorch.is_batchedtensor(q) and _lib.available())


# ----------------------------------------------------------------------------- ring attention in one launch
_HEADER = 256            # bytes of flag words in front of the staged tensors


def _ring_block(ar: Any, tag: tuple, nbytes: int) -> Any:
    """The next block of the two-deep staging ring ``tag`` (:meth:`symm.PeerArena.ring_block`)."""
    return ar.ring_block(tag, nbytes)


def _local_parts(blk: Any, P: int, base: int, slot: int, inner: int) -> Any:
    """Pointers to one operand (at ``inner`` inside a slot) in each of the ``P`` slots of this rank's block."""
    arr = (ctypes.c_void_p * 8)()
    for i in range(P):
        arr[i] = blk.ptr + base + i * slot + inner
    return arr


def _flag_ptrs(blk: Any, P: int, me: int) -> Any:
    arr = (ctypes.c_void_p * 8)()
    for i in range(P):
        arr[i] = None if i == me else blk.ptr + 4 * i
    return arr


class _RingFlashAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, group: Any) -> torch.Tensor:
        L, dev = _lib.lib(), q.device
        ar = symm.arena(dev)
        P, me = group.size(), group.rank()
        ranks = dist.get_process_group_ranks(group)
        s = q.shape[-2]
        q3 = q.reshape(-1, s, 64).contiguous()
        bh = q3.shape[0]
        n = bh * s * 64 * 2                                   # bytes of one staged operand
        slot = 2 * n                                          # K and V of one rank
        blk = _ring_block(ar, ("ring_fwd", dev.index, bh, s, tuple(ranks)), _HEADER + P * slot)
        mine = blk.tensor[_HEADER + me * slot:_HEADER + (me + 1) * slot].view(torch.bfloat16).view(2, *k.shape)
        mine[0].copy_(k)                                      # any strides (e.g. a head-transposed view): one copy
        mine[1].copy_(v)
        epoch, stride, replay, pushed = symm.push_slot_to_peers(ar, blk, ranks, me, _HEADER + me * slot, slot)
        out = torch.empty_like(q3)
        lse = torch.empty(bh, s, dtype=torch.float32, device=dev)
        rc = L.jb_flash_attn_fwd_parts(
            ctypes.c_void_p(q3.data_ptr()), _local_parts(blk, P, _HEADER, slot, 0), _local_parts(blk, P, _HEADER, slot, n),
            _flag_ptrs(blk, P, me), epoch, stride, replay, P, me, ctypes.c_void_p(out.data_ptr()),
            ctypes.c_void_p(lse.data_ptr()), bh, s, s, 64, s * 64, 64, s * 64, 64, s * 64, float(scale),
            ctypes.c_void_p(ar.status.data_ptr()), _lib.stream_ptr())
        torch.cuda.current_stream(dev).wait_event(pushed)
        if rc != 0:
            raise RuntimeError(f"jigsaw_b200 kernel launcher flash_attn_fwd_parts failed with code {rc}")
        _lib.count_launches(1)
        ctx.save_for_backward(q3, k, v, out, lse)
        ctx.scale, ctx.group, ctx.shape = float(scale), group, q.shape
        return out.view(q.shape)

    @staticmethod
    def backward(ctx: Any, g: torch.Tensor) -> tuple:
        q3, k, v, out, lse = ctx.saved_tensors
        group = ctx.group
        L, dev = _lib.lib(), q3.device
        ar = symm.arena(dev)
        P, me = group.size(), group.rank()
        ranks = dist.get_process_group_ranks(group)
        bh, s, _ = q3.shape
        n = bh * s * 64 * 2
        nf = bh * s * 4
        slot = 4 * n + 2 * nf                                  # q, dO, k, v, lse, D of one rank
        blk = _ring_block(ar, ("ring_bwd", dev.index, bh, s, tuple(ranks)), _HEADER + P * slot)
        base = _HEADER + me * slot
        ops = blk.tensor[base:base + 4 * n].view(torch.bfloat16).view(4, bh, s, 64)
        rows = blk.tensor[base + 4 * n:base + slot].view(torch.float32).view(2, bh, s)
        ops[0].copy_(q3)
        ops[1].view(ctx.shape).copy_(g)
        ops[2].view(ctx.shape).copy_(k)
        ops[3].view(ctx.shape).copy_(v)
        rows[0].copy_(lse)
        P_ = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
        rc = L.jb_flash_attn_delta(P_(out), P_(ops[1]), P_(rows[1]), bh * s, _lib.stream_ptr())
        if rc != 0:
            raise RuntimeError(f"jigsaw_b200 kernel launcher flash_attn_delta failed with code {rc}")
        epoch, stride, replay, pushed = symm.push_slot_to_peers(ar, blk, ranks, me, base, slot)
        dq, dk, dv = (torch.empty(bh, s, 64, dtype=torch.bfloat16, device=dev) for _ in range(3))
        at = lambda i: _local_parts(blk, P, _HEADER, slot, i * n)  # noqa: E731
        rc = L.jb_flash_attn_bwd_parts(
            P_(ops[0]), P_(ops[2]), P_(ops[3]), P_(ops[1]), at(0), at(1), _local_parts(blk, P, _HEADER, slot, 4 * n),
            _local_parts(blk, P, _HEADER, slot, 4 * n + nf), at(2), at(3), _flag_ptrs(blk, P, me), epoch, stride, replay, P, me,
            P_(dq), P_(dk), P_(dv), bh, s, ctx.scale, ctypes.c_void_p(ar.status.data_ptr()), _lib.stream_ptr())
        torch.cuda.current_stream(dev).wait_event(pushed)
        if rc != 0:
            raise RuntimeError(f"jigsaw_b200 kernel launcher flash_attn_bwd_parts failed with code {rc}")
        _lib.count_launches(3)
        return dq.view(ctx.shape), dk.view(ctx.shape), dv.view(ctx.shape), None, None


@_lib.traced("jb.maybe_fused_ring_attention")
@_lib.audited("ring_attention")
def maybe_fused_ring_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, group: Any,
                               dropout_p: float = 0.0) -> torch.Tensor | None:
    """Attention of the local queries ``(..., h, s, 64)`` against the keys / values of every rank of
    ``group`` (each holding ``s`` positions), differentiable, on the multi-part tcgen05 kernels; ``None``
    when they do not apply (then the chunked schedule of ``modules/attention/_ring.py`` runs)."""
    if not q.is_cuda:
        return None
    if group is None or not 2 <= group.size() <= 8:
        return _lib.decline("the group must have 2 to 8 ranks")
    if not flash_usable(q, k, dropout_p) or v.dtype != torch.bfloat16:
        return _lib.decline("needs bf16 operands with head dimension 64 and no dropout")
    if q.shape != k.shape or k.shape != v.shape or q.shape[-2] % 8:
        return _lib.decline("needs equal shapes of q, k, v on every rank and a local sequence that is a multiple of 8")
    return _RingFlashAttention.apply(q, k, v, scale, group)
