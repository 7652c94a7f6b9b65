"""Deferred execution of consecutive fused convolutions written as ordinary layers.

``nn.Sequential(DistributedConv2d, nn.GELU, DistributedConv2d, ...)`` is what a user (or
``convert_to_jigsaw``) builds.  Run layer by layer, every convolution would pack its input into the
padded channels-last layout, write a dense output and leave the activation to a separate kernel.
Instead an eligible ``DistributedConv2d`` returns a :class:`LazyConvChain`: a tensor subclass that
carries the metadata of the result (shape, dtype, device) but has not been computed yet.

* ``F.gelu`` of a lazy result marks the activation on the chain's last layer and stays lazy;
* the next eligible ``DistributedConv2d`` appends itself to the chain and stays lazy;
* anything else that touches the tensor (a loss, a norm, arithmetic, printing) materialises it: the
  whole chain then runs as ONE fused call (``conv_fused.conv_chain``): every layer's epilogue applies
  bias and activation, writes the next layer's padded input and pushes the halo to the neighbours,
  and the weight gradients are summed over the tile ranks under the backward pass.

The result is the same tensor the layer-by-layer path gives; only the schedule differs.

Reference parity: the layer API of jigsaw/modules/convolution/_conv/base.py:628-688 (one halo exchange,
one cuDNN call and one activation kernel per layer there).
"""

from __future__ import annotations

from typing import Any

import torch
import torch.nn.functional as F
from torch.utils._pytree import tree_map


def _getter(name: str) -> Any:
    return getattr(torch.Tensor, name).__get__


# Calls that only read metadata: answered by the wrapper itself, without running the chain.
_METADATA = {
    _getter("shape"), _getter("dtype"), _getter("device"), _getter("is_cuda"), _getter("ndim"), _getter("layout"),
    _getter("requires_grad"), _getter("is_sparse"), _getter("is_quantized"), _getter("is_meta"), _getter("is_cpu"),
    _getter("names"), _getter("is_nested"),
    torch.Tensor.dim, torch.Tensor.size, torch.Tensor.numel, torch.Tensor.element_size, torch.Tensor.is_floating_point,
    torch.Tensor.is_complex, torch.Tensor.ndimension, torch.Tensor.nelement, torch.Tensor.get_device,
}


class LazyConvChain(torch.Tensor):
    """Result of a chain of fused convolutions that has not run yet (see the module docstring)."""

    @staticmethod
    def __new__(cls, source: torch.Tensor, layers: tuple, acts: tuple, shape: tuple, grad_mode: bool, runner: Any) -> "LazyConvChain":
        return torch.Tensor._make_wrapper_subclass(cls, shape, dtype=torch.bfloat16, device=source.device, requires_grad=False)

    def __init__(self, source: torch.Tensor, layers: tuple, acts: tuple, shape: tuple, grad_mode: bool, runner: Any) -> None:
        self.source, self.layers, self.acts = source, tuple(layers), tuple(acts)
        self.grad_mode, self.runner = grad_mode, runner
        self._value: torch.Tensor | None = None

    # ------------------------------------------------------------------ building
    def with_activation(self) -> "LazyConvChain":
        return LazyConvChain(self.source, self.layers, self.acts[:-1] + (True,), tuple(self.shape), self.grad_mode, self.runner)

    def extended(self, layer: Any, act: bool, shape: tuple) -> "LazyConvChain":
        return LazyConvChain(self.source, self.layers + (layer,), self.acts + (act,), shape, self.grad_mode, self.runner)

    @property
    def pending(self) -> bool:
        return self._value is None

    # ------------------------------------------------------------------ running
    def materialize(self) -> torch.Tensor:
        """Run the chain (once) and return the real tensor."""
        if self._value is None:
            with torch.set_grad_enabled(self.grad_mode):
                self._value = self.runner(self.source, self.layers, self.acts)
        return self._value

    def __repr__(self) -> str:      # printing must not recurse through __torch_function__
        state = "pending" if self._value is None else "materialized"
        return f"LazyConvChain({len(self.layers)} layers, shape={tuple(self.shape)}, {state})"

    @classmethod
    def __torch_function__(cls, func: Any, types: Any, args: tuple = (), kwargs: dict | None = None) -> Any:
        kwargs = kwargs or {}
        if func in _METADATA:
            with torch._C.DisableTorchFunctionSubclass():
                return func(*args, **kwargs)
        if (func is F.gelu and len(args) == 1 and isinstance(args[0], LazyConvChain) and args[0].pending
                and not args[0].acts[-1] and kwargs.get("approximate", "none") == "none"):
            return args[0].with_activation()
        real = lambda t: t.materialize() if isinstance(t, LazyConvChain) else t  # noqa: E731
        args, kwargs = tree_map(real, (args, kwargs))
        with torch._C.DisableTorchFunctionSubclass():
            return func(*args, **kwargs)

    @classmethod
    def __torch_dispatch__(cls, func: Any, types: Any, args: tuple = (), kwargs: dict | None = None) -> Any:
        # safety net for calls that reach the dispatcher without passing __torch_function__: compute, then run
        real = lambda t: t.materialize() if isinstance(t, LazyConvChain) else t  # noqa: E731
        args, kwargs = tree_map(real, (args, kwargs or {}))
        return func(*args, **kwargs)


def materialize(x: Any) -> Any:
    """``x`` itself, or the computed tensor if ``x`` is a pending :class:`LazyConvChain`."""
    return x.materialize() if isinstance(x, LazyConvChain) else x
