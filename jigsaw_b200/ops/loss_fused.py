"""Fused squared-error loss (``csrc/elementwise.cu``): one kernel sums ``(input - target)^2`` over
tensors of any strides (the bf16 channels-last output of a fused convolution chain against an
fp32 NCHW target, for instance) and one writes the gradient with the strides and dtype of the
input, so nothing is copied, cast or re-laid-out between the model and the loss.

Reference parity: ``F.mse_loss(reduction="sum")`` in
jigsaw/modules/loss/_regression/functional.py:23-28 (ATen elementwise + reduce there).
"""

from __future__ import annotations

import ctypes
from typing import Any

import torch

from . import _lib

_OK = (torch.float32, torch.bfloat16)


def _order(a: torch.Tensor) -> list[int]:
    """Dimension order that walks ``a`` in memory order (largest stride first), so that the kernel's
    innermost loop index is contiguous in ``a``."""
    return sorted(range(a.dim()), key=lambda i: (-a.stride(i), i))


def _desc(t: torch.Tensor, order: list[int]) -> "_lib.JbStrided4":
    d = _lib.JbStrided4()
    d.ptr, d.is_bf16 = t.data_ptr(), int(t.dtype == torch.bfloat16)
    pad = 4 - t.dim()
    for i in range(4):
        d.stride[i] = 0 if i < pad else t.stride(order[i - pad])
    return d


def _sizes(t: torch.Tensor, order: list[int]):
    pad = 4 - t.dim()
    return (ctypes.c_int * 4)(*([1] * pad + [t.shape[i] for i in order]))


_scratch: dict[int, tuple[torch.Tensor, torch.Tensor]] = {}


def _scratch_for(dev: torch.device) -> tuple[torch.Tensor, torch.Tensor]:
    if dev.index not in _scratch:
        _scratch[dev.index] = (torch.empty(_lib.sm_count(dev.index) * 8, dtype=torch.float32, device=dev),
                               torch.zeros(1, dtype=torch.int32, device=dev))
    return _scratch[dev.index]


def _dense(t: torch.Tensor) -> bool:
    """True when the elements of ``t`` tile one block of memory without gaps or overlaps (any
    dimension order)."""
    expect = 1
    for size, stride in sorted(((sz, st) for sz, st in zip(t.shape, t.stride()) if sz != 1), key=lambda p: p[1]):
        if stride != expect:
            return False
        expect *= size
    return True


PAIR_OPS = {"mse": 0, "l1": 1, "smooth_l1": 2, "bce": 3, "bce_logits": 4}


class _PairLossSum(torch.autograd.Function):
    """``sum f(a, b)`` over all elements for one of the element-wise losses of ``PAIR_OPS``."""

    @staticmethod
    def forward(ctx: Any, a: torch.Tensor, b: torch.Tensor, op: int, beta: float) -> torch.Tensor:
        L, dev = _lib.lib(), a.device
        partial, counter = _scratch_for(dev)
        out = torch.empty((), dtype=torch.float32, device=dev)
        order = _order(a)
        da, db = _desc(a, order), _desc(b, order)
        rc = L.jb_pair_loss_sum(ctypes.byref(da), ctypes.byref(db), _sizes(a, order), op, float(beta),
                                ctypes.c_void_p(partial.data_ptr()), ctypes.c_void_p(counter.data_ptr()),
                                ctypes.c_void_p(out.data_ptr()), _lib.sm_count(dev.index), _lib.stream_ptr())
        if rc != 0:
            raise RuntimeError(f"jigsaw_b200 kernel launcher pair_loss_sum failed with code {rc}")
        _lib.count_launches(1)
        ctx.save_for_backward(a, b)
        ctx.op, ctx.beta = op, float(beta)
        return out

    @staticmethod
    def backward(ctx: Any, g: torch.Tensor) -> tuple:
        a, b = ctx.saved_tensors
        L, dev = _lib.lib(), a.device
        ga = gb = None
        scale = g.float().contiguous()
        if ctx.needs_input_grad[0]:
            ga = torch.empty_strided(a.shape, a.stride(), dtype=a.dtype, device=dev)
            order = _order(a)
            da, db = _desc(a, order), _desc(b, order)
            rc = L.jb_pair_loss_grad(ctypes.byref(da), ctypes.byref(db), _sizes(a, order), ctx.op, ctx.beta,
                                     ctypes.c_void_p(scale.data_ptr()), ctypes.c_void_p(ga.data_ptr()),
                                     int(ga.dtype == torch.bfloat16), _lib.sm_count(dev.index), _lib.stream_ptr())
            if rc != 0:
                raise RuntimeError(f"jigsaw_b200 kernel launcher pair_loss_grad failed with code {rc}")
            _lib.count_launches(1)
        if ctx.needs_input_grad[1]:
            if ctx.op != 0:
                raise NotImplementedError("only the squared error is differentiable in its target on the fused path")
            gb = (-2.0 * scale) * (a.float() - b.float()).to(b.dtype)
        return ga, gb, None, None


@_lib.traced("jb.maybe_fused_sq_diff_sum")
@_lib.audited("sq_diff_sum")
def maybe_fused_sq_diff_sum(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor | None:
    """``sum((a - b)^2)`` as an fp32 scalar (differentiable in ``a``), or ``None`` when the
    kernel does not apply."""
    return _pair_loss_sum(a, b, "mse", 1.0)


@_lib.traced("jb.maybe_fused_pair_loss_sum")
@_lib.audited("pair_loss_sum")
def maybe_fused_pair_loss_sum(a: torch.Tensor, b: torch.Tensor, kind: str, beta: float = 1.0) -> torch.Tensor | None:
    """``sum f(a, b)`` as an fp32 scalar, differentiable in ``a``, for ``kind`` in ``"l1"``, ``"smooth_l1"``
    (with ``beta``), ``"bce"`` (``a`` holds probabilities), ``"bce_logits"`` (``a`` holds logits); one kernel
    per direction on tensors of any strides; ``None`` when the kernel does not apply."""
    return _pair_loss_sum(a, b, kind, beta)


def _pair_loss_sum(a: torch.Tensor, b: torch.Tensor, kind: str, beta: float) -> torch.Tensor | None:
    if not a.is_cuda:
        return None
    if a.shape == b.shape and a.dim() > 4 and a.is_contiguous() and b.is_contiguous():
        a, b = a.reshape(-1), b.reshape(-1)          # volumes and the like: element-wise, so one long row will do
    if a.shape != b.shape or a.dim() > 4 or a.dim() == 0 or a.numel() == 0:
        return _lib.decline("needs two tensors of the same shape with 1 to 4 dimensions")
    if a.dtype not in _OK or b.dtype not in _OK or torch._C._functorch.is_batchedtensor(a):
        return _lib.decline("needs fp32 or bf16 tensors outside vmap")
    if b.requires_grad and kind != "mse":
        return _lib.decline("the target needs a gradient")
    if kind == "smooth_l1" and not beta > 0.0:
        return _lib.decline("smooth L1 with beta = 0 is the absolute error")
    # the gradient is written with the strides of ``a``: they must address distinct elements
    if not _dense(a):
        return _lib.decline("the prediction overlaps itself in memory")
    if not _lib.available():
        raise RuntimeError("jigsaw_b200: the sm_100a kernel library is missing on a CUDA machine")
    return _PairLossSum.apply(a, b, PAIR_OPS[kind], float(beta))


# ----------------------------------------------------------------------------- cross-entropy
class _CrossEntropyRows(torch.autograd.Function):
    """Per-row softmax cross-entropy of logits ``[B, C_local, S]`` whose class dimension is split
    over ``group`` (``csrc/norm.cu``): one kernel computes the local (max, sum-exp, true-class logit),
    exchanges them with the other class shards through peer memory and finishes the row."""

    @staticmethod
    def forward(ctx: Any, x: torch.Tensor, target: torch.Tensor, group: Any, ignore_index: int) -> torch.Tensor:
        from .norm_fused import _Exchange
        from . import symm

        L, dev = _lib.lib(), x.device
        B, C, S = x.shape
        R = B * S
        sm = _lib.sm_count(dev.index)
        grid = L.jb_cross_entropy_grid(B, C, S, sm)
        loss = torch.empty(R, dtype=torch.float32, device=dev)
        lse = torch.empty(R, dtype=torch.float32, device=dev)
        lo = 0 if group is None else group.rank() * C
        ex = _Exchange(dev, group, R, grid, width=4, kind="cross_entropy")
        rc = L.jb_cross_entropy_fwd(ctypes.c_void_p(x.data_ptr()), int(x.dtype == torch.bfloat16),
                                    ctypes.c_void_p(target.data_ptr()), ignore_index, B, C, S, lo,
                                    ctypes.c_void_p(loss.data_ptr()), ctypes.c_void_p(lse.data_ptr()), ctypes.byref(ex.desc),
                                    ctypes.c_void_p(symm.arena(dev).status.data_ptr()), sm, _lib.stream_ptr())
        ex.done()
        if rc != 0:
            raise RuntimeError(f"jigsaw_b200 kernel launcher cross_entropy_fwd failed with code {rc}")
        _lib.count_launches(1)
        ctx.save_for_backward(x, target, lse)
        ctx.lo, ctx.ignore = lo, ignore_index
        return loss

    @staticmethod
    def backward(ctx: Any, g: torch.Tensor) -> tuple:
        x, target, lse = ctx.saved_tensors
        L, dev = _lib.lib(), x.device
        B, C, S = x.shape
        dx = torch.empty_like(x)
        grow = g.float().contiguous()
        rc = L.jb_cross_entropy_bwd(ctypes.c_void_p(x.data_ptr()), int(x.dtype == torch.bfloat16),
                                    ctypes.c_void_p(target.data_ptr()), ctx.ignore, B, C, S, ctx.lo,
                                    ctypes.c_void_p(lse.data_ptr()), ctypes.c_void_p(grow.data_ptr()),
                                    ctypes.c_void_p(dx.data_ptr()), int(dx.dtype == torch.bfloat16), _lib.sm_count(dev.index),
                                    _lib.stream_ptr())
        if rc != 0:
            raise RuntimeError(f"jigsaw_b200 kernel launcher cross_entropy_bwd failed with code {rc}")
        _lib.count_launches(1)
        return dx, None, None, None


@_lib.traced("jb.maybe_fused_cross_entropy")
@_lib.audited("cross_entropy")
def maybe_fused_cross_entropy(logits: torch.Tensor, target: torch.Tensor, dim: int, channel_group: Any,
                              ignore_index: int) -> torch.Tensor | None:
    """Unreduced cross-entropy (shape of ``target``, fp32, zero where ignored) for index targets,
    or ``None`` when the kernel does not apply."""
    if not logits.is_cuda or logits.dtype not in _OK or target.dtype != torch.int64 or logits.numel() == 0:
        return None
    if logits.dim() < 2 or torch._C._functorch.is_batchedtensor(logits):
        return None
    parts = 1 if channel_group is None else channel_group.size()
    if parts > 8 or logits.numel() >= 2 ** 31:
        return None
    if not _lib.available():
        raise RuntimeError("jigsaw_b200: the sm_100a kernel library is missing on a CUDA machine")
    shape = logits.shape
    B = 1
    for n in shape[:dim]:
        B *= n
    S = 1
    for n in shape[dim + 1:]:
        S *= n
    x = logits.contiguous().view(B, shape[dim], S)
    rows = _CrossEntropyRows.apply(x, target.contiguous().view(-1), channel_group if parts > 1 else None, int(ignore_index))
    return rows.view(target.shape)
