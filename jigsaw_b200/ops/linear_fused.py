"""Linear layers on the tcgen05 GEMM kernel (``csrc/gemm.cu``).

``maybe_fused_linear(x, w, b)`` computes ``x @ w.T + b`` under bf16 autocast (or for bf16
inputs) with the persistent TMA + TMEM kernel: bias (and optionally GELU) are applied in the
epilogue, and the backward pass runs the two other products from the *stored* tensors, without
transposing anything: ``dX = dY @ W`` (B operand MN-major) and ``dW = dY.T @ X`` (both operands
MN-major, fp32 output).  Returns ``None`` when the kernel does not apply; the caller then uses
``torch.nn.functional.linear``.

Reference parity: the ``torch.matmul`` / ``F.linear`` calls of
jigsaw/modules/linear/_distributed_matmul.py:100-110,159-177 (cuBLAS there).
"""

from __future__ import annotations

import ctypes
from typing import Any

import torch

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
