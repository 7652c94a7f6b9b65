"""Attention helpers on the GPU: the online-softmax merge of ring-attention chunks
(``csrc/elementwise.cu``), one launch instead of half a dozen elementwise kernels.

Reference parity: the Triton merge kernel of
jigsaw/modules/attention/_merge_kernel.py:37-82 (launch :140-163), here as a CUDA kernel.
"""

from __future__ import annotations

import ctypes

import torch

from . import _lib


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
    Forward only (no autograd): the cores of ``jigsaw_b200.modules.attention`` do not call it yet, because
    the kernel has not run on hardware; ``tests/test_elementwise_gpu.py`` holds its numerics test, which
    runs when ``JIGSAW_FLASH_ATTENTION=1`` is set.

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
        from . import symm

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
    (``csrc/flash_attn.cu``, ``csrc/flash_attn_bwd.cu``); same shapes as :func:`flash_attention_forward`.
    Not called by the attention layers unless ``JIGSAW_FLASH_ATTENTION=1`` (the kernels have not run on
    hardware)."""

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
