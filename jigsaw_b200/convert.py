"""In-place conversion of a plain PyTorch model into its distributed counterpart.

Conversion is plan-then-apply: :class:`ConversionPlan` decides, in one flat pass over
``named_modules`` and before anything is touched, what happens to every module (replace, keep,
report, block); ``apply`` then builds the replacements deepest-first and re-binds them on their
parents.  Exact-type matches of ``mapped_modules`` are replaced through the class method
``convert_to_jigsaw`` of the distributed layer; ``container_converters`` replace a whole sub-tree
(``Attention``); ``shard_safe_modules`` (elementwise) stay as they are; ``shard_unsafe_modules``
(anything that reduces over, mixes along or reshapes a dimension that may be sharded) block the
conversion unless ``non_safe=True``; everything else is reported according to ``on_unrecognized``.
Extra keyword arguments (``comm=``, ``ring=``, ``ulysses=``, ``dim_to_mesh_axis=`` ...) are forwarded
to every layer converter.

Reference parity: jigsaw/convert.py:20-38 (tables), :41-171 (safe / unsafe lists),
:174-209 (pre-flight walk), :212-315 (convert_to_jigsaw), :318-371 (recursive worker).
"""

from __future__ import annotations

import warnings
from collections.abc import Callable
from dataclasses import dataclass
from typing import Any, Literal

import torch
from torch import nn

from .modules import activation, attention, convolution, linear, normalization, roll

__all__ = [
    "ConversionPlan",
    "convert_to_jigsaw",
    "mapped_modules",
    "container_converters",
    "shard_safe_modules",
    "shard_unsafe_modules",
]

mapped_modules: dict[type[nn.Module], Any] = {
    nn.Linear: linear.DistributedLinear,
    nn.Conv1d: convolution.DistributedConv1d,
    nn.Conv2d: convolution.DistributedConv2d,
    nn.Conv3d: convolution.DistributedConv3d,
    nn.ConvTranspose1d: convolution.DistributedConvTranspose1d,
    nn.ConvTranspose2d: convolution.DistributedConvTranspose2d,
    nn.ConvTranspose3d: convolution.DistributedConvTranspose3d,
    roll.Roll: roll.DistributedRoll,
    nn.LayerNorm: normalization.DistributedLayerNorm,
    nn.GroupNorm: normalization.DistributedGroupNorm,
    nn.Softmax: activation.DistributedSoftmax,
    linear.MatMulXWT: linear.DistributedMatMulXWT,
    linear.MatMulXW: linear.DistributedMatMulXW,
    linear.MatMulXTW: linear.DistributedMatMulXTW,
}

container_converters: dict[type[nn.Module], Callable[..., nn.Module]] = {
    attention.Attention: attention.Attention.convert_to_jigsaw,
}

#: Elementwise modules: correct on any shard.
shard_safe_modules: tuple[type[nn.Module], ...] = (
    nn.Identity, nn.ReLU, nn.ReLU6, nn.LeakyReLU, nn.ELU, nn.SELU, nn.CELU, nn.GELU, nn.SiLU, nn.Mish, nn.Sigmoid,
    nn.Tanh, nn.Hardtanh, nn.Hardsigmoid, nn.Hardswish, nn.Softplus, nn.Dropout, nn.Dropout1d, nn.Dropout2d,
    nn.Dropout3d, nn.AlphaDropout,
)


def _existing(*names: str) -> tuple[type[nn.Module], ...]:
    return tuple(getattr(nn, n) for n in names if hasattr(nn, n))


#: Modules that reduce over, mix along or reshape dimensions: wrong on a shard of that dimension.
shard_unsafe_modules: tuple[type[nn.Module], ...] = _existing(
    "Softmax", "Softmax2d", "Softmin", "LogSoftmax", "AdaptiveLogSoftmaxWithLoss", "GLU", "PReLU",
    "BatchNorm1d", "BatchNorm2d", "BatchNorm3d", "LazyBatchNorm1d", "LazyBatchNorm2d", "LazyBatchNorm3d",
    "SyncBatchNorm", "InstanceNorm1d", "InstanceNorm2d", "InstanceNorm3d", "LazyInstanceNorm1d",
    "LazyInstanceNorm2d", "LazyInstanceNorm3d", "RMSNorm", "LocalResponseNorm", "CrossMapLRN2d",
    "MaxPool1d", "MaxPool2d", "MaxPool3d", "MaxUnpool1d", "MaxUnpool2d", "MaxUnpool3d", "AvgPool1d", "AvgPool2d",
    "AvgPool3d", "FractionalMaxPool2d", "FractionalMaxPool3d", "LPPool1d", "LPPool2d", "LPPool3d",
    "AdaptiveMaxPool1d", "AdaptiveMaxPool2d", "AdaptiveMaxPool3d", "AdaptiveAvgPool1d", "AdaptiveAvgPool2d",
    "AdaptiveAvgPool3d", "ZeroPad1d", "ZeroPad2d", "ZeroPad3d", "ConstantPad1d", "ConstantPad2d", "ConstantPad3d",
    "ReflectionPad1d", "ReflectionPad2d", "ReflectionPad3d", "ReplicationPad1d", "ReplicationPad2d",
    "ReplicationPad3d", "CircularPad1d", "CircularPad2d", "CircularPad3d", "Flatten", "Unflatten", "Fold", "Unfold",
    "PixelShuffle", "PixelUnshuffle", "ChannelShuffle", "Upsample", "UpsamplingNearest2d", "UpsamplingBilinear2d",
    "CosineSimilarity", "PairwiseDistance", "Embedding", "EmbeddingBag", "Bilinear", "LazyLinear", "LazyConv1d",
    "LazyConv2d", "LazyConv3d", "LazyConvTranspose1d", "LazyConvTranspose2d", "LazyConvTranspose3d", "RNNBase",
    "RNNCellBase", "MultiheadAttention", "Transformer", "TransformerEncoder", "TransformerDecoder",
    "TransformerEncoderLayer", "TransformerDecoderLayer",
) + (nn.modules.loss._Loss,)


def _is_ours(m: nn.Module) -> bool:
    mod = type(m).__module__
    return mod.startswith("jigsaw_b200.") or mod.startswith("jigsaw.")


# ----------------------------------------------------------------------------- plan, then apply
@dataclass
class _Step:
    """What happens to one module of the tree."""

    path: str                      # dotted name ("" = the root)
    module: nn.Module
    action: str                    # "replace" | "keep" | "report" | "block"
    reason: str = ""
    maker: Callable[..., nn.Module] | None = None


class ConversionPlan:
    """The decision for every module of ``model``, made in ONE flat pass over ``named_modules`` before
    anything is touched.  A module is settled by the first rule that applies, and a settled module settles
    its whole sub-tree (the pass skips every path below it):

    1. exact type in ``container_converters`` or ``mapped_modules``  -> replace (built by the layer's
       ``convert_to_jigsaw``);
    2. already a layer of this library                              -> keep;
    3. instance of ``shard_unsafe_modules``                          -> block (conversion refuses unless ``non_safe``);
    4. a leaf: elementwise (``shard_safe_modules``) -> keep, otherwise -> report;
    5. a container: descend; if it owns parameters itself           -> also report.

    ``apply`` then builds the replacements and re-binds them on their parents, deepest paths first, so a
    replaced child never invalidates a path still to be visited."""

    def __init__(self, model: nn.Module, convert_layer_norm: bool = True) -> None:
        self.model = model
        self.steps: list[_Step] = []
        settled: list[str] = []
        for path, module in model.named_modules():
            if any(path == root or path.startswith(root + ".") for root in settled if root) or "" in settled:
                continue
            step = self._decide(path, module, convert_layer_norm)
            if step is None:
                continue                                     # a plain container: its children are visited next
            self.steps.append(step)
            if step.action != "report" or not any(True for _ in module.children()):
                settled.append(path)

    @staticmethod
    def _decide(path: str, module: nn.Module, convert_layer_norm: bool) -> _Step | None:
        kind = type(module)
        skip_norm = isinstance(module, nn.LayerNorm) and not convert_layer_norm
        if kind in container_converters:
            return _Step(path, module, "replace", maker=container_converters[kind])
        if kind in mapped_modules and not skip_norm:
            return _Step(path, module, "replace", maker=mapped_modules[kind].convert_to_jigsaw)
        if skip_norm or _is_ours(module):
            return _Step(path, module, "keep")
        if isinstance(module, shard_unsafe_modules):
            return _Step(path, module, "block", f"non-elementwise module {kind.__name__}")
        if not any(True for _ in module.children()):
            if isinstance(module, shard_safe_modules):
                return _Step(path, module, "keep")
            return _Step(path, module, "report", f"unrecognized leaf module {kind.__name__}")
        if any(True for _ in module.parameters(recurse=False)):
            return _Step(path, module, "report", f"{kind.__name__} owns parameters directly, which are not sharded")
        return None

    def findings(self, action: str) -> list[tuple[str, str]]:
        return [(s.path or "<root>", s.reason) for s in self.steps if s.action == action]

    def apply(self, mesh: dict, device: Any, keys: dict, kwargs: dict) -> nn.Module:
        root = self.model
        for step in sorted((s for s in self.steps if s.action == "replace"), key=lambda s: -s.path.count(".")):
            new = step.maker(step.module, mesh, device, **keys, **kwargs)
            if step.path == "":
                root = new
                continue
            parent_path, _, name = step.path.rpartition(".")
            setattr(root.get_submodule(parent_path) if parent_path else root, name, new)
        return root


def convert_to_jigsaw(
    model: nn.Module,
    process_mesh_dict: dict,
    device: torch.device | str,
    row_kw: str = "row",
    col_kw: str = "col",
    model_kw: str = "model",
    convert_layer_norm: bool = True,
    on_unrecognized: Literal["warn", "raise", "ignore"] = "warn",
    non_safe: bool = False,
    **kwargs: Any,
) -> nn.Module:
    """Convert ``model`` in place (the same container is returned; a bare convertible layer
    is returned as its replacement).  Use the same seed on every rank so that all ranks
    slice the same global weights.  Nothing is modified if the pre-flight check fails."""
    if on_unrecognized not in ("warn", "raise", "ignore"):
        raise ValueError(f"on_unrecognized must be 'warn', 'raise' or 'ignore', got {on_unrecognized!r}")
    plan = ConversionPlan(model, convert_layer_norm)
    blocked = plan.findings("block")
    if blocked and not non_safe:
        raise ValueError(
            "convert_to_jigsaw has no distributed version of these modules; as plain torch they compute on "
            "the local shard only and give wrong results if the dimension they reduce over, mix along or "
            "reshape is sharded. Pass non_safe=True if it is not:\n" + "\n".join(f"  {n}: {r}" for n, r in blocked)
        )
    left_alone = blocked + plan.findings("report")
    if left_alone and on_unrecognized != "ignore":
        msg = (
            "convert_to_jigsaw leaves these modules as plain torch; they compute on the local shard only, "
            "which is wrong if they reduce over or mix along a sharded dimension:\n"
            + "\n".join(f"  {n}: {r}" for n, r in left_alone)
        )
        if on_unrecognized == "raise":
            raise ValueError(msg)
        warnings.warn(msg, stacklevel=2)
    return plan.apply(process_mesh_dict, device, dict(row_kw=row_kw, col_kw=col_kw, model_kw=model_kw), kwargs)
