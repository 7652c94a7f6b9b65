"""Optimizers on the package's own kernels.

:class:`FusedAdam` updates all fp32 CUDA parameters of a group in one multi-tensor launch
(``csrc/elementwise.cu``) instead of a handful of elementwise kernels per parameter.  The step
counter lives on the device and is advanced by a one-thread kernel, so the whole update can sit
inside a CUDA graph (:class:`jigsaw_b200.utils.GraphedStep`).  Parameters that are not fp32 CUDA
tensors take the plain PyTorch formulas.

:func:`fused_grad_norm` computes the global gradient norm of many tensors in one launch (a
deterministic two-level reduction), for gradient clipping.

Reference parity: the reference trains with ``torch.optim`` (examples/vit.py:244); the optimizer
step is one of the "remaining hot ops" of its benchmark configurations.
"""

from __future__ import annotations

import ctypes
from collections.abc import Iterable

import torch

from .ops import _lib

_MAX = 48


def _table(params, grads, ms, vs) -> "_lib.JbAdamTensors":
    t = _lib.JbAdamTensors()
    t.count = len(params)
    for i, (p, g, m, v) in enumerate(zip(params, grads, ms, vs)):
        t.p[i] = p.data_ptr()
        t.g[i] = g.data_ptr()
        t.m[i] = 0 if m is None else m.data_ptr()
        t.v[i] = 0 if v is None else v.data_ptr()
        t.numel[i] = p.numel()
    return t


class FusedAdam(torch.optim.Optimizer):
    """Adam (``decoupled_weight_decay=False``) or AdamW (``True``) with bias correction.

    ``lr`` may be a one-element fp32 tensor on the parameters' device: the kernel then reads it from
    memory at every step, so a schedule can change it (``group["lr"].fill_(x)``) between replays of a
    CUDA graph that captured the step.

    Step counting on the fused path: ONE device counter per parameter group and device, advanced once per
    ``step()`` call; every parameter of the group takes its bias correction from it.  ``torch.optim.Adam``
    (and the plain path of this class) count per parameter, so a parameter whose gradient was ``None`` in some
    steps (frozen for a while, an unused branch) is corrected here as if it had taken part in every step of its
    group.  Put such parameters into a group of their own if the difference matters.  The correction terms
    ``1 - beta ** step`` are evaluated in fp32 with the fast-math power function: at step 1 with
    ``beta2 = 0.999`` the relative deviation from the exact value is about 2e-4, and it vanishes as the
    step count grows."""

    def __init__(self, params: Iterable, lr: float = 1e-3, betas: tuple[float, float] = (0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.0, decoupled_weight_decay: bool = False, maximize: bool = False) -> None:
        if float(lr) < 0 or eps < 0 or not 0 <= betas[0] < 1 or not 0 <= betas[1] < 1 or weight_decay < 0:
            raise ValueError("invalid Adam hyper-parameter")
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                                      decoupled_weight_decay=decoupled_weight_decay, maximize=maximize))

    @torch.no_grad()
    def step(self, closure=None, grad_scale: torch.Tensor | None = None):
        """One update.  ``grad_scale`` (optional device scalar) multiplies every gradient first
        (the factor of a gradient-norm clip)."""
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            fused, plain = [], []
            for p in group["params"]:
                if p.grad is None:
                    continue
                if p.grad.is_sparse:
                    raise RuntimeError("FusedAdam does not support sparse gradients")
                st = self.state[p]
                if not st:
                    st["exp_avg"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                    st["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                ok = (p.is_cuda and p.dtype == torch.float32 and p.grad.dtype == torch.float32 and p.is_contiguous()
                      and p.grad.is_contiguous() and _lib.available())
                (fused if ok else plain).append(p)
            b1, b2 = group["betas"]
            by_device: dict[torch.device, list] = {}
            for p in fused:
                by_device.setdefault(p.device, []).append(p)
            for dev, ps in by_device.items():
                key = ("step", dev)
                if key not in group:
                    group[key] = torch.zeros((), dtype=torch.float32, device=dev)
                step = group[key]
                L = _lib.lib()
                with torch.cuda.device(dev):
                    st_ptr = _lib.stream_ptr()
                    L.jb_increment(ctypes.c_void_p(step.data_ptr()), st_ptr)
                    for i in range(0, len(ps), _MAX):
                        chunk = ps[i:i + _MAX]
                        tab = _table(chunk, [p.grad for p in chunk], [self.state[p]["exp_avg"] for p in chunk],
                                     [self.state[p]["exp_avg_sq"] for p in chunk])
                        tail = (b1, b2, group["eps"], group["weight_decay"], int(group["decoupled_weight_decay"]),
                                int(group["maximize"]), ctypes.c_void_p(step.data_ptr()),
                                None if grad_scale is None else ctypes.c_void_p(grad_scale.data_ptr()), st_ptr)
                        lr = group["lr"]
                        if torch.is_tensor(lr):
                            # a device scalar: a schedule may overwrite it between replays of a captured step
                            if lr.device != dev or lr.dtype != torch.float32 or lr.numel() != 1:
                                raise ValueError("a tensor learning rate must be one fp32 value on the parameters' device")
                            rc = L.jb_adam_multi_lr(ctypes.byref(tab), ctypes.c_void_p(lr.data_ptr()), *tail)
                        else:
                            rc = L.jb_adam_multi(ctypes.byref(tab), lr, *tail)
                        if rc != 0:
                            raise RuntimeError(f"jigsaw_b200 kernel launcher adam_multi failed with code {rc}")
                    _lib.count_launches(1 + (len(ps) + _MAX - 1) // _MAX)
            for p in plain:
                st = self.state[p]
                st["step"] = st.get("step", 0) + 1
                g = p.grad if grad_scale is None else p.grad * grad_scale.to(p.grad.device)
                g = -g if group["maximize"] else g
                if group["weight_decay"]:
                    if group["decoupled_weight_decay"]:
                        p.mul_(1 - float(group["lr"]) * group["weight_decay"])
                    else:
                        g = g.add(p, alpha=group["weight_decay"])
                st["exp_avg"].mul_(b1).add_(g, alpha=1 - b1)
                st["exp_avg_sq"].mul_(b2).addcmul_(g, g, value=1 - b2)
                c1, c2 = 1 - b1 ** st["step"], 1 - b2 ** st["step"]
                p.addcdiv_(st["exp_avg"], (st["exp_avg_sq"] / c2).sqrt_().add_(group["eps"]), value=-float(group["lr"]) / c1)
        return loss


def fused_grad_norm(grads: Iterable[torch.Tensor]) -> torch.Tensor:
    """``sqrt(sum_i ||g_i||^2)`` of fp32 CUDA tensors on one device as a device scalar, in
    ``ceil(n / 48)`` launches; other tensors are added with PyTorch."""
    grads = [g for g in grads if g is not None]
    if not grads:
        return torch.zeros(())
    dev = grads[0].device
    total = torch.zeros((), dtype=torch.float32, device=dev)
    ok = [g for g in grads if g.is_cuda and g.device == dev and g.dtype == torch.float32 and g.is_contiguous()]
    rest = [g for g in grads if not any(g is o for o in ok)]
    if ok and _lib.available():
        L = _lib.lib()
        counter = torch.zeros(1, dtype=torch.int32, device=dev)
        with torch.cuda.device(dev):
            for i in range(0, len(ok), _MAX):
                chunk = ok[i:i + _MAX]
                partial = torch.empty(sum(L.jb_chunks(g.numel()) for g in chunk), dtype=torch.float32, device=dev)
                tab = _table(chunk, chunk, [None] * len(chunk), [None] * len(chunk))
                rc = L.jb_sumsq_multi(ctypes.byref(tab), ctypes.c_void_p(partial.data_ptr()),
                                      ctypes.c_void_p(counter.data_ptr()), ctypes.c_void_p(total.data_ptr()),
                                      _lib.stream_ptr())
                if rc != 0:
                    raise RuntimeError(f"jigsaw_b200 kernel launcher sumsq_multi failed with code {rc}")
            _lib.count_launches((len(ok) + _MAX - 1) // _MAX)
    else:
        rest = grads
    for g in rest:
        total = total + g.float().pow(2).sum().to(dev)
    return total.sqrt()
