"""Linear layers on the tcgen05 GEMM kernel (``csrc/gemm.cu``).

``maybe_fused_linear(x, w, b)`` computes ``x @ w.T + b`` under bf16 autocast (or for bf16
inputs) with the persistent TMA + TMEM kernel: bias (and optionally GELU) are applied in the
epilogue, and the backward pass runs the two other products from the *stored* tensors, without
transposing anything: ``dX = dY @ W`` (B operand MN-major) and ``dW = dY.T @ X`` (both operands
MN-major, fp32 output).  Returns ``None`` when the kernel does not apply; the caller then uses
``torch.nn.functional.linear``.

``maybe_fused_gather_linear(x_local, w, b, group)`` overlaps the all-gather of the activations
with that GEMM: every rank writes its ``[M, K / P]`` block (cast to bf16) into its slot of a symmetric
buffer, the copy engines push the slot into every peer's buffer followed by a flag, and the TMA
producer of the GEMM reads the k-blocks of part ``p`` from LOCAL memory as soon as the flag of rank
``p`` has arrived, so the transfer (each byte crosses NVLink once per destination, no SM involved) runs
under the tensor-core work on the parts that are already there.  The input gradient is GEMM ->
reduce-scatter in one pass: the epilogue of ``dY @ W`` stores each tile into the inbox of the rank that
owns those columns, and every rank sums the slabs it received.  The weight gradient multiplies with the
gathered activations saved by the forward pass (no second gather).

Reference parity: the ``torch.matmul`` / ``F.linear`` calls of
jigsaw/modules/linear/_distributed_matmul.py:100-110,159-177 (cuBLAS there) and the masked
all-to-alls that move ``x`` blocks before them (jigsaw/_core/comm.py:430-455).
"""

from __future__ import annotations

import ctypes
from typing import Any

import torch
import torch.distributed as dist

from . import _lib, symm


def _p(t: torch.Tensor | None) -> ctypes.c_void_p | None:
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False, bias: torch.Tensor | None = None,
         gelu: bool = False, out_dtype: torch.dtype = torch.bfloat16, out: torch.Tensor | None = None,
         accumulate: bool = False) -> torch.Tensor:
    """``act(A @ B + bias)`` for bf16 matrices stored row-major.

    ``a`` is ``[M, K]`` (``a_mn=False``) or ``[K, M]`` (``a_mn=True``); ``b`` is ``[N, K]``
    (``b_mn=False``) or ``[K, N]`` (``b_mn=True``).  Row strides must be multiples of 8 elements.
    """
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        raise TypeError("gemm operands must be bf16")
    if a.stride(-1) != 1 or b.stride(-1) != 1:
        raise ValueError("gemm operands must have a contiguous last dimension")
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    if K != Kb:
        raise ValueError(f"reduction sizes differ: {K} vs {Kb}")
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=a.device)
    dev = a.device
    rc = _lib.lib().jb_gemm_bf16(_p(a), _p(b), _p(out), _p(bias), M, N, K, a.stride(0), b.stride(0), out.stride(0),
                                 int(a_mn), int(b_mn), int(gelu), int(out.dtype == torch.float32), int(accumulate),
                                 _lib.sm_count(dev.index), _p(symm.arena(dev).status), _lib.stream_ptr())
    if rc != 0:
        raise RuntimeError(f"jigsaw_b200 kernel launcher gemm_bf16 failed with code {rc}")
    _lib.count_launches(1)
    return out


class _FusedLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None) -> torch.Tensor:
        K = x.shape[-1]
        xb = x.reshape(-1, K)
        xb = xb if xb.dtype == torch.bfloat16 else xb.to(torch.bfloat16)
        xb = xb if xb.is_contiguous() else xb.contiguous()
        wb = w if w.dtype == torch.bfloat16 else w.to(torch.bfloat16)
        wb = wb if wb.is_contiguous() else wb.contiguous()
        bias = None if b is None else b.float().contiguous()
        y = gemm(xb, wb, bias=bias)
        ctx.save_for_backward(xb, wb)
        ctx.has_bias, ctx.x_shape, ctx.x_dtype, ctx.w_dtype = b is not None, x.shape, x.dtype, w.dtype
        ctx.b_dtype = None if b is None else b.dtype
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx: Any, gy: torch.Tensor) -> tuple:
        xb, wb = ctx.saved_tensors
        N = wb.shape[0]
        g = gy.reshape(-1, N)
        g = g if g.dtype == torch.bfloat16 else g.to(torch.bfloat16)
        g = g if g.is_contiguous() else g.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(g, wb, b_mn=True).view(ctx.x_shape).to(ctx.x_dtype)          # [M, N] x [N, K]
        if ctx.needs_input_grad[1]:
            dw = gemm(g, xb, a_mn=True, b_mn=True, out_dtype=torch.float32).to(ctx.w_dtype)   # [M, N]^T x [M, K]
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = g.sum(dim=0, dtype=torch.float32).to(ctx.b_dtype)
        return dx, dw, db


@_lib.traced("jb.maybe_fused_linear")
@_lib.audited("linear")
def maybe_fused_linear(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None) -> torch.Tensor | None:
    if not x.is_cuda or w.dim() != 2 or x.numel() == 0:
        return None
    bf16 = x.dtype == torch.bfloat16 or (torch.is_autocast_enabled("cuda") and torch.get_autocast_dtype("cuda") == torch.bfloat16)
    if not bf16 or x.dtype not in (torch.float32, torch.bfloat16) or w.dtype not in (torch.float32, torch.bfloat16):
        return None
    N, K = w.shape
    M = x.numel() // K
    if K % 8 or N % 8 or M % 8 or K < 64 or N < 16 or torch._C._functorch.is_batchedtensor(x):
        return None
    if not _lib.available():
        raise RuntimeError("jigsaw_b200: the sm_100a kernel library is missing on a CUDA machine")
    return _FusedLinear.apply(x, w, b)


class _FusedMatmul(torch.autograd.Function):
    """``op(a) @ op(b)`` for 2-D operands (``op`` = transpose when the flag is set) on the tcgen05 GEMM, which reads
    either operand in either major order: no transposed copy in the forward or in the two gradient products."""

    @staticmethod
    def forward(ctx: Any, a: torch.Tensor, b: torch.Tensor, a_t: bool, b_t: bool) -> torch.Tensor:
        ab = (a if a.dtype == torch.bfloat16 else a.to(torch.bfloat16)).contiguous()
        bb = (b if b.dtype == torch.bfloat16 else b.to(torch.bfloat16)).contiguous()
        ctx.save_for_backward(ab, bb)
        ctx.a_t, ctx.b_t, ctx.a_dtype, ctx.b_dtype = a_t, b_t, a.dtype, b.dtype
        return gemm(ab, bb, a_mn=a_t, b_mn=not b_t)

    @staticmethod
    def backward(ctx: Any, gy: torch.Tensor) -> tuple:
        ab, bb = ctx.saved_tensors
        g = (gy if gy.dtype == torch.bfloat16 else gy.to(torch.bfloat16)).contiguous()      # [M, N]
        da = db = None
        if ctx.needs_input_grad[0]:
            if ctx.a_t:      # a is [K, M]: da = op(b) g^T
                da = gemm(bb, g, a_mn=ctx.b_t, b_mn=False, out_dtype=torch.float32)
            else:            # a is [M, K]: da = g op(b)^T
                da = gemm(g, bb, a_mn=False, b_mn=ctx.b_t, out_dtype=torch.float32)
            da = da.to(ctx.a_dtype)
        if ctx.needs_input_grad[1]:
            if ctx.b_t:      # b is [N, K]: db = g^T op(a)
                db = gemm(g, ab, a_mn=True, b_mn=not ctx.a_t, out_dtype=torch.float32)
            else:            # b is [K, N]: db = op(a)^T g
                db = gemm(ab, g, a_mn=not ctx.a_t, b_mn=True, out_dtype=torch.float32)
            db = db.to(ctx.b_dtype)
        return da, db, None, None


@_lib.traced("jb.maybe_fused_matmul")
@_lib.audited("matmul")
def maybe_fused_matmul(a: torch.Tensor, b: torch.Tensor, a_t: bool = False, b_t: bool = False) -> torch.Tensor | None:
    """``op(a) @ op(b)`` for 2-D operands under bf16 autocast (or for bf16 operands) on the tcgen05 GEMM, differentiable;
    ``None`` when it does not apply."""
    if not a.is_cuda or a.dim() != 2 or b.dim() != 2 or a.numel() == 0 or b.numel() == 0:
        return None
    bf16 = (a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16) or (
        torch.is_autocast_enabled("cuda") and torch.get_autocast_dtype("cuda") == torch.bfloat16)
    if not bf16 or a.dtype not in (torch.float32, torch.bfloat16) or b.dtype not in (torch.float32, torch.bfloat16):
        return _lib.decline("needs bf16 numerics")
    M, K = (a.shape[1], a.shape[0]) if a_t else a.shape
    N = b.shape[0] if b_t else b.shape[1]
    if K % 8 or N % 8 or M % 8 or K < 64 or N < 16 or torch._C._functorch.is_batchedtensor(a):
        return _lib.decline("needs M, N, K multiples of 8, K >= 64 and N >= 16")
    return _FusedMatmul.apply(a, b, a_t, b_t)


# ----------------------------------------------------------------------------- all-gather -> GEMM
_HEADER = 256          # bytes of flag words in front of the staged block


def _staging_block(ar: "symm.PeerArena", tag: tuple, nbytes: int) -> "symm.Block":
    """The next block of the two-deep staging ring ``tag`` (:meth:`symm.PeerArena.ring_block`)."""
    return ar.ring_block(tag, nbytes)


def scatter_gemm_launcher(L: Any) -> Any:
    """Scatter GEMM whose tiles leave through shared memory as 128-byte row pieces: the form that suits
    stores into a peer's memory (row-per-thread stores reach about 160 GB/s across NVLink)."""
    return L.jb_gemm_bf16_scatter_staged


def _scatter_gemm(g: torch.Tensor, wb: torch.Tensor, group: Any) -> torch.Tensor:
    """``reduce_scatter(g @ wb, last dim over group)`` with the scatter fused into the GEMM: the
    epilogue stores every tile of column part ``p`` straight into rank ``p``'s inbox (this rank's
    slab), a flag follows, and each rank sums the ``P`` slabs of its inbox."""
    L, dev = _lib.lib(), g.device
    ar = symm.arena(dev)
    P, me = group.size(), group.rank()
    ranks = dist.get_process_group_ranks(group)
    M, N = g.shape
    K = wb.shape[1]
    kp = K // P
    slab = M * kp * 2
    blk = _staging_block(ar, ("scatter_dx", dev.index, M, kp, tuple(ranks)), _HEADER + P * slab)
    epoch = ar.next_own_epoch(blk)
    stride = ar.capture_stride or 0
    replay = ar.replay.data_ptr() if ar.capture_stride is not None else None
    st = _lib.stream_ptr()
    c_part = (ctypes.c_void_p * 8)()
    for i, r in enumerate(ranks):
        c_part[i] = (blk.ptr if i == me else blk.peer_ptr(r)) + _HEADER + me * slab
    rc = scatter_gemm_launcher(L)(_p(g), _p(wb), c_part, P, kp, M, N, g.stride(0), wb.stride(0), 0, 1,
                                _lib.sm_count(dev.index), _p(ar.status), st)
    flags = (ctypes.c_void_p * 8)()
    n = 0
    for i, r in enumerate(ranks):
        if i != me:
            flags[n] = blk.peer_ptr(r) + 4 * me
            n += 1
    if rc == 0:
        rc = L.jb_publish(flags, n, epoch, stride, replay, st)
    waits = (ctypes.c_void_p * 8)()
    for i in range(P):
        waits[i] = None if i == me else blk.ptr + 4 * i
    out = torch.empty(M, kp, dtype=torch.bfloat16, device=dev)
    if rc == 0:
        rc = L.jb_sum_slabs(ctypes.c_void_p(blk.ptr + _HEADER), M * kp, P, waits, epoch, stride, replay, _p(out), 1,
                            _p(ar.status), _lib.sm_count(dev.index), st)
    if rc != 0:
        raise RuntimeError(f"jigsaw_b200 kernel launcher gemm_bf16_scatter failed with code {rc}")
    _lib.count_launches(3)
    return out


class _GatherLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None, group: Any) -> torch.Tensor:
        L, dev = _lib.lib(), x.device
        ar = symm.arena(dev)
        P, me = group.size(), group.rank()
        ranks = dist.get_process_group_ranks(group)
        kp = x.shape[-1]
        M = x.numel() // kp
        N = w.shape[0]
        K = P * kp
        # the gathered [M, K] matrix lives in every rank's block: this rank writes its own column block (cast + copy
        # in one kernel) and the copy engines push it into the same columns of every peer, followed by a flag; the
        # GEMM then reads ALL parts from local memory as their flags arrive, so each activation byte crosses NVLink
        # once per destination
        blk = _staging_block(ar, ("gather_x", dev.index, M, kp, tuple(ranks)), _HEADER + M * K * 2)
        full = blk.tensor[_HEADER:_HEADER + M * K * 2].view(torch.bfloat16).view(M, K)
        full[:, me * kp:(me + 1) * kp].copy_(x.reshape(M, kp))
        epoch, stride, replay, pushed = symm.push_slot_to_peers(ar, blk, ranks, me, _HEADER + me * kp * 2, kp * 2,
                                                                pitch=K * 2, rows=M)
        st = _lib.stream_ptr()
        g = _lib.JbGather()
        for i in range(P):
            g.a_part[i] = blk.ptr + _HEADER + i * kp * 2
            g.flag[i] = None if i == me else blk.ptr + 4 * i
        g.epoch, g.stride, g.replay, g.parts, g.k_part, g.lda_part = epoch, stride, replay, P, kp, K
        wb = w if w.dtype == torch.bfloat16 else w.to(torch.bfloat16)
        wb = wb if wb.is_contiguous() else wb.contiguous()
        bias = None if b is None else b.float().contiguous()
        y = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        rc = L.jb_gemm_bf16_gather(ctypes.byref(g), _p(wb), _p(y), _p(bias), M, N, wb.stride(0), y.stride(0), 0, 0,
                                   _lib.sm_count(dev.index), _p(ar.status), st)
        torch.cuda.current_stream(dev).wait_event(pushed)
        if rc != 0:
            raise RuntimeError(f"jigsaw_b200 kernel launcher gemm_bf16_gather failed with code {rc}")
        _lib.count_launches(1)
        # the weight gradient needs the gathered activations: keep a copy of the complete block (every part has
        # arrived once the GEMM is done) instead of gathering again in the backward pass
        ctx.save_for_backward(full.clone() if ctx.needs_input_grad[1] else None, wb)
        ctx.group, ctx.x_shape, ctx.x_dtype, ctx.w_dtype = group, x.shape, x.dtype, w.dtype
        ctx.b_dtype = None if b is None else b.dtype
        return y.view(*x.shape[:-1], N)

    @staticmethod
    def backward(ctx: Any, gy: torch.Tensor) -> tuple:
        x_full, wb = ctx.saved_tensors
        group = ctx.group
        N = wb.shape[0]
        g = gy.reshape(-1, N)
        g = g if g.dtype == torch.bfloat16 else g.to(torch.bfloat16)
        g = g if g.is_contiguous() else g.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = _scatter_gemm(g, wb, group).view(ctx.x_shape).to(ctx.x_dtype)
        if ctx.needs_input_grad[1]:
            dw = gemm(g, x_full, a_mn=True, b_mn=True, out_dtype=torch.float32).to(ctx.w_dtype)   # [M, N]^T x [M, K]
        if ctx.b_dtype is not None and ctx.needs_input_grad[2]:
            db = g.sum(dim=0, dtype=torch.float32).to(ctx.b_dtype)
        return dx, dw, db, None


@_lib.traced("jb.maybe_fused_gather_linear")
@_lib.audited("gather_linear")
def maybe_fused_gather_linear(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None, group: Any) -> torch.Tensor | None:
    """``all_gather(x over group, last dim) @ w.T + b`` in one GEMM whose producer reads the other
    ranks' blocks from their memory, or ``None`` when that does not apply.  ``w`` is ``[N, K]``
    with ``K = group.size() * x.shape[-1]``."""
    if group is None or group.size() < 2 or group.size() > 8 or not x.is_cuda or w.dim() != 2 or x.numel() == 0:
        return None
    bf16 = x.dtype == torch.bfloat16 or (torch.is_autocast_enabled("cuda") and torch.get_autocast_dtype("cuda") == torch.bfloat16)
    if not bf16 or x.dtype not in (torch.float32, torch.bfloat16) or w.dtype not in (torch.float32, torch.bfloat16):
        return None
    kp = x.shape[-1]
    N, K = w.shape
    M = x.numel() // kp
    if K != kp * group.size() or kp % 64 or N % 8 or M % 8 or N < 16 or torch._C._functorch.is_batchedtensor(x):
        return None
    if not _lib.available():
        raise RuntimeError("jigsaw_b200: the sm_100a kernel library is missing on a CUDA machine")
    return _GatherLinear.apply(x, w, b, group)
