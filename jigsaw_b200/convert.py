"""In-place conversion of a plain PyTorch model into its distributed counterpart.

The converter walks the module tree once *before* touching anything and classifies every
module: exact-type matches of ``mapped_modules`` are replaced by the class method
``convert_to_jigsaw`` of the distributed layer; ``container_converters`` replace a whole
sub-tree (``Attention``); ``shard_safe_modules`` (elementwise) stay as they are;
``shard_unsafe_modules`` (anything that reduces over, mixes along or reshapes a dimension
that may be sharded) abort the conversion unless ``non_safe=True``; everything else is
reported according to ``on_unrecognized``.  Extra keyword arguments (``comm=``, ``ring=``,
``ulysses=``, ``dim_to_mesh_axis=`` ...) are forwarded to every layer converter.

Reference parity: jigsaw/convert.py:20-38 (tables), :41-171 (safe / unsafe lists),
:174-209 (pre-flight walk), :212-315 (convert_to_jigsaw), :318-371 (recursive worker).
"""

from __future__ import annotations

import warnings
from collections.abc import Callable, Iterator
from typing import Any, Literal

import torch
from torch import nn

from .modules import activation, attention, convolution, linear, normalization, roll

__all__ = [
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


def _preflight(model: nn.Module, prefix: str, convert_layer_norm: bool) -> Iterator[tuple[str, str, bool]]:
    """``(qualified name, reason, unsafe)`` for every module the converter will leave alone."""
    name = prefix or "<root>"
    kind = type(model)
    if kind in container_converters or kind in mapped_modules:
        if not (kind is nn.LayerNorm and not convert_layer_norm):
            return
    if isinstance(model, nn.LayerNorm) and not convert_layer_norm:
        return
    if _is_ours(model):
        return
    if isinstance(model, shard_unsafe_modules):
        yield name, f"non-elementwise module {kind.__name__}", True
        return
    children = list(model.named_children())
    if not children:
        if not isinstance(model, shard_safe_modules):
            yield name, f"unrecognized leaf module {kind.__name__}", False
        return
    if any(True for _ in model.parameters(recurse=False)):
        yield name, f"{kind.__name__} owns parameters directly, which are not sharded", False
    for child_name, child in children:
        yield from _preflight(child, f"{prefix}.{child_name}" if prefix else child_name, convert_layer_norm)


def _walk_and_replace(model: nn.Module, mesh: dict, device: Any, convert_layer_norm: bool, keys: dict, kwargs: dict) -> nn.Module:
    kind = type(model)
    if kind in container_converters:
        return container_converters[kind](model, mesh, device, **keys, **kwargs)
    if kind in mapped_modules and not (kind is nn.LayerNorm and not convert_layer_norm):
        return mapped_modules[kind].convert_to_jigsaw(model, mesh, device, **keys, **kwargs)
    if _is_ours(model):
        return model
    for child_name, child in list(model.named_children()):
        new = _walk_and_replace(child, mesh, device, convert_layer_norm, keys, kwargs)
        if new is not child:
            setattr(model, child_name, new)
    return model


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
    found = list(_preflight(model, "", convert_layer_norm))
    unsafe = [(n, r) for n, r, bad in found if bad]
    if unsafe and not non_safe:
        raise ValueError(
            "convert_to_jigsaw has no distributed version of these modules; as plain torch they compute on "
            "the local shard only and give wrong results if the dimension they reduce over, mix along or "
            "reshape is sharded. Pass non_safe=True if it is not:\n" + "\n".join(f"  {n}: {r}" for n, r in unsafe)
        )
    if found and on_unrecognized != "ignore":
        msg = (
            "convert_to_jigsaw leaves these modules as plain torch; they compute on the local shard only, "
            "which is wrong if they reduce over or mix along a sharded dimension:\n"
            + "\n".join(f"  {n}: {r}" for n, r, _ in found)
        )
        if on_unrecognized == "raise":
            raise ValueError(msg)
        warnings.warn(msg, stacklevel=2)
    keys = dict(row_kw=row_kw, col_kw=col_kw, model_kw=model_kw)
    return _walk_and_replace(model, process_mesh_dict, device, convert_layer_norm, keys, kwargs)
