"""Softmax and log-softmax along a dimension that may be split over GPUs, on the fused kernels.

Forward: one launch computes every row's log-sum-exp (local maximum and sum of exponentials, exchanged
with the other class shards through peer memory inside the kernel, ``csrc/norm.cu`` ``ce_fwd_kernel``
without targets), one element-wise launch writes ``x - lse`` or ``exp(x - lse)``.  Backward: one launch
for the row sums the gradient needs (``sum g`` or ``sum g y``), the peer-memory all-reduce kernel over the
class shards, one element-wise launch for ``dx``.  No library collective is involved.

Reference parity: jigsaw/modules/activation/_functional.py:23-91 (softmax: MAX then SUM all-reduce forward,
SUM backward), :94-177 (log-softmax).
"""

from __future__ import annotations

import ctypes
from typing import Any

import torch
import torch.distributed as dist

from . import _lib, symm


def _p(t: torch.Tensor | None) -> ctypes.c_void_p | None:
    return None if t is None else ctypes.c_void_p(t.data_ptr())


class _FusedSoftmax(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, x: torch.Tensor, dim: int, group: Any, log: bool, out_dtype: torch.dtype) -> torch.Tensor:
        from .norm_fused import _Exchange

        L, dev = _lib.lib(), x.device
        x = x.contiguous()
        B = 1
        for n in x.shape[:dim]:
            B *= n
        C = x.shape[dim]
        S = x.numel() // (B * C)
        R = B * S
        sm = _lib.sm_count(dev.index)
        grid = L.jb_cross_entropy_grid(B, C, S, sm)
        lse = torch.empty(R, dtype=torch.float32, device=dev)
        ex = _Exchange(dev, group, R, grid, width=4, kind="cross_entropy")
        rc = L.jb_cross_entropy_fwd(_p(x), int(x.dtype == torch.bfloat16), None, -100, B, C, S, 0, None, _p(lse),
                                    ctypes.byref(ex.desc), _p(symm.arena(dev).status), sm, _lib.stream_ptr())
        ex.done()
        y = torch.empty(x.shape, dtype=out_dtype, device=dev)
        if rc == 0:
            rc = L.jb_softmax_apply(_p(x), int(x.dtype == torch.bfloat16), _p(lse), _p(y), int(out_dtype == torch.bfloat16),
                                    B, C, S, int(log), sm, _lib.stream_ptr())
        if rc != 0:
            raise RuntimeError(f"jigsaw_b200 kernel launcher softmax failed with code {rc}")
        _lib.count_launches(2)
        ctx.save_for_backward(y)
        ctx.geom, ctx.group, ctx.log, ctx.x_dtype = (B, C, S), group, log, x.dtype
        return y

    @staticmethod
    def backward(ctx: Any, g: torch.Tensor) -> tuple:
        from . import reduce_fused

        (y,) = ctx.saved_tensors
        L, dev = _lib.lib(), y.device
        B, C, S = ctx.geom
        sm = _lib.sm_count(dev.index)
        g = g.contiguous()
        if g.dtype not in (torch.float32, torch.bfloat16):
            g = g.float()
        d = torch.empty(B * S, dtype=torch.float32, device=dev)
        rc = L.jb_softmax_rowdot(_p(y), int(y.dtype == torch.bfloat16), _p(g), int(g.dtype == torch.bfloat16), _p(d), B, C, S,
                                 int(ctx.log), sm, _lib.stream_ptr())
        if rc == 0 and ctx.group is not None and ctx.group.size() > 1:
            if not reduce_fused.maybe_fused_all_reduce([d], dist.get_process_group_ranks(ctx.group)):
                dist.all_reduce(d, group=ctx.group)
        dx = torch.empty(y.shape, dtype=ctx.x_dtype, device=dev)
        if rc == 0:
            rc = L.jb_softmax_bwd(_p(y), int(y.dtype == torch.bfloat16), _p(g), int(g.dtype == torch.bfloat16), _p(d), _p(dx),
                                  int(dx.dtype == torch.bfloat16), B, C, S, int(ctx.log), sm, _lib.stream_ptr())
        if rc != 0:
            raise RuntimeError(f"jigsaw_b200 kernel launcher softmax backward failed with code {rc}")
        _lib.count_launches(2)
        return dx, None, None, None, None


@_lib.traced("jb.maybe_fused_softmax")
@_lib.audited("softmax")
def maybe_fused_softmax(x: torch.Tensor, dim: int, group: Any, log: bool) -> torch.Tensor | None:
    """``softmax`` / ``log_softmax`` of ``x`` along ``dim`` (split over ``group``, or local when ``None``): fp32
    result under autocast, else the input dtype; ``None`` when the kernels do not apply."""
    if not x.is_cuda:
        return None
    if x.dtype not in (torch.float32, torch.bfloat16) or x.numel() == 0 or torch._C._functorch.is_batchedtensor(x):
        return _lib.decline("needs fp32 or bf16 input outside vmap")
    if group is not None and group.size() > 8:
        return _lib.decline("at most 8 class shards")
    if x.numel() >= 2 ** 31:
        return _lib.decline("tensor too large for 32-bit row arithmetic")
    if not _lib.available():
        raise RuntimeError("jigsaw_b200: the sm_100a kernel library is missing on a CUDA machine")
    out_dtype = torch.float32 if torch.is_autocast_enabled("cuda") else x.dtype
    return _FusedSoftmax.apply(x, dim % x.dim(), group, log, out_dtype)
