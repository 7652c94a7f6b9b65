"""Attention cores with an explicit forward / backward contract, and the online-softmax merge.

    forward (q, k, v, scale, dropout_p, seed)            -> (out, lse, rng_state)
    backward(dout, q, k, v, out, lse, scale, dropout_p, rng_state) -> (dq, dk, dv)

Layout ``(..., heads, seq, head_dim)``.  ``lse`` is the row-wise log-sum-exp in fp32.  The
backward takes the FINAL (merged) ``out`` and ``lse`` of the whole ring, which makes every
chunk's gradient exact: ``P = exp(S - lse)`` are the true global probabilities.

``math`` is the unfused reference (any device / dtype, seeded dropout); ``sdpa`` calls the
flash-attention kernels bundled with PyTorch and falls back to ``math`` on CPU.

Reference parity: jigsaw/modules/attention/_functional/cores/math.py:31-149,
cores/sdpa.py:17-165, forward.py:23-61 and _merge_kernel.py:37-172 (merge).
"""

from __future__ import annotations

from typing import Any

import torch


def chunk_seed(base_seed: int, rank: int, chunk: int) -> int:
    """Per-(rank, chunk) dropout seed, reproducible between forward and backward."""
    return (base_seed ^ (rank * 1_000_003) ^ (chunk * 999_999_937)) % (2**31 - 1)


def _dropout_mask(shape: torch.Size, p: float, seed: int, device: torch.device) -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    return (torch.rand(shape, generator=g, device=device) >= p).to(torch.float32) / (1.0 - p)


class MathCore:
    """Unfused ``softmax(q k^T) v`` in fp32 accumulation."""

    name = "math"

    @staticmethod
    def forward(q, k, v, scale: float, dropout_p: float = 0.0, seed: int = 0) -> tuple[torch.Tensor, torch.Tensor, Any]:
        acc = torch.promote_types(q.dtype, torch.float32)
        s = torch.matmul(q.to(acc), k.to(acc).transpose(-1, -2)) * scale
        lse = torch.logsumexp(s, dim=-1)
        p = torch.exp(s - lse.unsqueeze(-1))
        if dropout_p > 0.0:
            p = p * _dropout_mask(p.shape, dropout_p, seed, p.device)
        out = torch.matmul(p, v.to(acc))
        return out.to(q.dtype), lse, seed

    @staticmethod
    def backward(dout, q, k, v, out, lse, scale: float, dropout_p: float = 0.0, rng_state: Any = 0):
        acc = torch.promote_types(q.dtype, torch.float32)
        qf, kf, vf, do = q.to(acc), k.to(acc), v.to(acc), dout.to(acc)
        p = torch.exp(torch.matmul(qf, kf.transpose(-1, -2)) * scale - lse.to(acc).unsqueeze(-1))
        delta = (do * out.to(acc)).sum(dim=-1, keepdim=True)
        dp = torch.matmul(do, vf.transpose(-1, -2))
        if dropout_p > 0.0:
            mask = _dropout_mask(p.shape, dropout_p, rng_state, p.device)
            dv = torch.matmul((p * mask).transpose(-1, -2), do)
            dp = dp * mask
        else:
            dv = torch.matmul(p.transpose(-1, -2), do)
        ds = p * (dp - delta)
        dq = torch.matmul(ds, kf) * scale
        dk = torch.matmul(ds.transpose(-1, -2), qf) * scale
        return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype)


class SdpaCore:
    """Flash-attention kernels of PyTorch (forward returns the LSE and the philox state)."""

    name = "sdpa"

    @staticmethod
    def _usable(q: torch.Tensor) -> bool:
        return q.is_cuda and q.dtype in (torch.float16, torch.bfloat16) and q.shape[-1] <= 256 and q.shape[-1] % 8 == 0

    @staticmethod
    def _4d(t: torch.Tensor) -> torch.Tensor:
        return t.reshape(-1, *t.shape[-3:]) if t.dim() != 4 else t

    @staticmethod
    def forward(q, k, v, scale: float, dropout_p: float = 0.0, seed: int = 0):
        if not SdpaCore._usable(q):
            return MathCore.forward(q, k, v, scale, dropout_p, seed)
        shape = q.shape
        res = torch.ops.aten._scaled_dot_product_flash_attention(
            SdpaCore._4d(q), SdpaCore._4d(k), SdpaCore._4d(v), dropout_p, False, False, scale=scale
        )
        out, lse, philox_seed, philox_offset = res[0], res[1], res[6], res[7]
        return out.reshape(shape), lse.reshape(shape[:-1]), (philox_seed, philox_offset)

    @staticmethod
    def backward(dout, q, k, v, out, lse, scale: float, dropout_p: float = 0.0, rng_state: Any = None):
        if not SdpaCore._usable(q) or not isinstance(rng_state, tuple):
            return MathCore.backward(dout, q, k, v, out, lse, scale, dropout_p, rng_state)
        f = SdpaCore._4d
        sq, sk = q.shape[-2], k.shape[-2]
        dq, dk, dv = torch.ops.aten._scaled_dot_product_flash_attention_backward(
            f(dout).contiguous(), f(q), f(k), f(v), f(out).to(q.dtype), lse.reshape(-1, *lse.shape[-2:]).float(),
            None, None, sq, sk, dropout_p, False, rng_state[0], rng_state[1], scale=scale,
        )
        return dq.reshape(q.shape), dk.reshape(k.shape), dv.reshape(v.shape)


class Tcgen05Core:
    """Own attention kernels for head dimension 64 (``ops/attention_fused.py``); anything they do not
    cover (other head sizes, dropout, non-bf16 data, CPU) goes to :class:`SdpaCore`.  The default core
    of every backend except ``math``."""

    name = "tcgen05"

    @staticmethod
    def _usable(q: torch.Tensor, k: torch.Tensor, dropout_p: float) -> bool:
        return (q.is_cuda and q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16 and q.shape[-1] == 64 and dropout_p == 0.0
                and q.shape[:-2] == k.shape[:-2] and not torch._C._functorch.is_batchedtensor(q))

    @staticmethod
    def forward(q, k, v, scale: float, dropout_p: float = 0.0, seed: int = 0):
        if not Tcgen05Core._usable(q, k, dropout_p):
            return SdpaCore.forward(q, k, v, scale, dropout_p, seed)
        from ...ops import attention_fused

        out, lse = attention_fused.flash_attention_forward(q, k, v, scale)
        return out, lse, "tcgen05"

    @staticmethod
    def backward(dout, q, k, v, out, lse, scale: float, dropout_p: float = 0.0, rng_state: Any = None):
        if rng_state != "tcgen05":
            return SdpaCore.backward(dout, q, k, v, out, lse, scale, dropout_p, rng_state)
        from ...ops import attention_fused

        return attention_fused.flash_attention_backward(dout, q, k, v, out, lse, scale)


def select_core(backend: Any) -> Any:
    name = getattr(backend, "value", backend)
    if name == "math":
        return MathCore
    return Tcgen05Core


def merge_chunks(out: torch.Tensor, lse: torch.Tensor, out_j: torch.Tensor, lse_j: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Online-softmax merge of a new chunk result into the running (fp32) state:
    ``out <- out + sigmoid(lse_j - lse) (out_j - out)``, ``lse <- logaddexp(lse, lse_j)``."""
    if out.is_cuda:
        from ...ops import attention_fused

        merged = attention_fused.maybe_fused_merge(out, lse, out_j, lse_j)
        if merged is not None:
            return merged
    w = torch.sigmoid(lse_j - lse).unsqueeze(-1)
    return out + w * (out_j.to(out.dtype) - out), torch.logaddexp(lse, lse_j)
