"""Attention helpers on the GPU: the online-softmax merge of ring-attention chunks
(``csrc/elementwise.cu``), one launch instead of half a dozen elementwise kernels.

Reference parity: the Triton merge kernel of
jigsaw/modules/attention/_merge_kernel.py:37-82 (launch :140-163), here as a CUDA kernel.
"""

from __future__ import annotations

import ctypes

import torch

from . import _lib


def __getattr__(name: str):
    if name.startswith("maybe_fused_"):
        return lambda *a, **k: None
    raise AttributeError(name)


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
