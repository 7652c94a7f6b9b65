"""Loss functions on sharded tensors: same value and gradient as the torch loss on the
gathered tensor, with only the terms that cross a shard boundary reduced.

Two kinds of sharding: ``channel_group`` splits the class dimension of a classification
input (log-softmax, true-class pick and label-smoothing term reduce over it);
``reduce_groups`` lists the groups splitting the remaining dimensions (only the final sum /
mean needs them; the mean divides by the GLOBAL normaliser).  The backward of the final
reduction is the identity: every rank seeds the same upstream gradient.

Reference parity: jigsaw/modules/loss/_common.py:41-190,
_classification/functional.py:22-400, _regression/functional.py:14-131, loss/README.md.
"""

from __future__ import annotations

from collections.abc import Sequence

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ..._core.collectives import reduce_from_group
from ..activation._functional import distributed_log_softmax

GroupsArg = "Sequence[dist.ProcessGroup | None] | dist.ProcessGroup | None"


def _groups(groups) -> tuple:
    if groups is None:
        return ()
    if isinstance(groups, dist.ProcessGroup):
        return (groups,)
    return tuple(groups)


def _gsize(g: dist.ProcessGroup | None) -> int:
    return 1 if g is None else g.size()


def _grank(g: dist.ProcessGroup | None) -> int:
    return 0 if g is None else g.rank()


def redundant_all_reduce(x: torch.Tensor, groups) -> torch.Tensor:
    """Sum ``x`` over ``groups``; the gradient passes through unchanged."""
    return reduce_from_group(x, _groups(groups))


def _check_reduction(reduction: str) -> None:
    if reduction not in ("none", "sum", "mean"):
        raise ValueError(f"{reduction} is not a valid value for reduction")


def reduce_scalar_loss(local_sum: torch.Tensor, local_denom: torch.Tensor, reduction: str, reduce_groups) -> torch.Tensor:
    """Global ``sum`` or ``mean`` from local numerator and normaliser, reduced in >= fp32."""
    groups = _groups(reduce_groups)
    acc = torch.promote_types(torch.promote_types(local_sum.dtype, local_denom.dtype), torch.float32)
    if reduction == "sum":
        return redundant_all_reduce(local_sum.to(acc), groups).to(local_sum.dtype)
    both = redundant_all_reduce(torch.stack((local_sum.to(acc), local_denom.to(acc))), groups)
    return (both[0] / both[1]).to(local_sum.dtype)


# ----------------------------------------------------------------------------- regression
_FUSED_PAIR_KINDS = {F.l1_loss: "l1", F.smooth_l1_loss: "smooth_l1", F.binary_cross_entropy: "bce",
                     F.binary_cross_entropy_with_logits: "bce_logits"}


def _elementwise_loss(fn, input, target, reduction, reduce_groups, **kw):
    _check_reduction(reduction)
    if reduction == "none":
        return fn(input, target, reduction="none", **kw)
    total = None
    if input.is_cuda and all(v is None for k, v in kw.items() if k != "beta"):
        from ...ops import loss_fused

        # one kernel per direction, any strides / bf16 input (weight and pos_weight stay on the torch path)
        if fn is F.mse_loss:
            total = loss_fused.maybe_fused_sq_diff_sum(input, target)
        elif fn in _FUSED_PAIR_KINDS and (fn is not F.smooth_l1_loss or kw.get("beta", 1.0) > 0.0):
            total = loss_fused.maybe_fused_pair_loss_sum(input, target, _FUSED_PAIR_KINDS[fn], kw.get("beta", 1.0))
    if total is None:
        with torch.autocast(input.device.type, enabled=False):
            acc = torch.promote_types(input.dtype, torch.float32)
            total = fn(input.to(acc), target.to(acc), reduction="sum", **kw)
    count = torch.full((), float(input.numel()), dtype=torch.float32, device=input.device)   # device-side fill: capturable
    # result dtype as in torch: the promotion of input and target (a bf16 prediction against an fp32 target gives fp32)
    return reduce_scalar_loss(total, count, reduction, reduce_groups).to(torch.promote_types(input.dtype, target.dtype))


def distributed_mse_loss(input, target, *, reduction: str = "mean", reduce_groups=None) -> torch.Tensor:
    """``F.mse_loss`` over a tensor sharded across ``reduce_groups``."""
    return _elementwise_loss(F.mse_loss, input, target, reduction, reduce_groups)


def distributed_l1_loss(input, target, *, reduction: str = "mean", reduce_groups=None) -> torch.Tensor:
    """``F.l1_loss`` over a tensor sharded across ``reduce_groups``."""
    return _elementwise_loss(F.l1_loss, input, target, reduction, reduce_groups)


def distributed_smooth_l1_loss(input, target, *, beta: float = 1.0, reduction: str = "mean", reduce_groups=None) -> torch.Tensor:
    """``F.smooth_l1_loss`` over a tensor sharded across ``reduce_groups``."""
    return _elementwise_loss(F.smooth_l1_loss, input, target, reduction, reduce_groups, beta=beta)


# ----------------------------------------------------------------------------- binary cross-entropy
def distributed_binary_cross_entropy(probs, target, *, weight=None, reduction: str = "mean", reduce_groups=None) -> torch.Tensor:
    """``F.binary_cross_entropy`` (probabilities in) over a sharded tensor.  ``reduce_groups``
    must list EVERY group the tensor is split over, the channel group included."""
    return _elementwise_loss(F.binary_cross_entropy, probs, target, reduction, reduce_groups, weight=weight)


def distributed_binary_cross_entropy_with_logits(
    logits, target, *, weight=None, pos_weight=None, reduction: str = "mean", reduce_groups=None
) -> torch.Tensor:
    """``F.binary_cross_entropy_with_logits`` over a sharded tensor (see the BCE note on groups)."""
    return _elementwise_loss(
        F.binary_cross_entropy_with_logits, logits, target, reduction, reduce_groups, weight=weight, pos_weight=pos_weight
    )


# ----------------------------------------------------------------------------- classification
def _pick_target(logp: torch.Tensor, target: torch.Tensor, dim: int, channel_group, ignore_index: int):
    """Per-element true-class log-probability (partial: non-zero only on the owning rank),
    the validity mask and the clamped local index."""
    c_local = logp.shape[dim]
    lo = _grank(channel_group) * c_local
    valid = target != ignore_index
    local = target - lo
    mine = valid & (local >= 0) & (local < c_local)
    idx = torch.where(mine, local, torch.zeros_like(local))
    picked = logp.gather(dim, idx.unsqueeze(dim)).squeeze(dim)
    picked = torch.where(mine, picked, torch.zeros_like(picked))
    return picked, valid


def distributed_nll_loss(
    log_probs, target, *, weight=None, ignore_index: int = -100, reduction: str = "mean", dim: int = 1,
    channel_group=None, reduce_groups=None,
) -> torch.Tensor:
    """``F.nll_loss`` on log-probabilities whose class dimension ``dim`` is split over
    ``channel_group``; ``weight`` has the GLOBAL class count and is replicated."""
    _check_reduction(reduction)
    dim = dim % log_probs.dim()
    in_dtype = log_probs.dtype
    logp = log_probs.to(torch.promote_types(in_dtype, torch.float32))
    picked, valid = _pick_target(logp, target, dim, channel_group, ignore_index)
    picked = redundant_all_reduce(picked, channel_group)
    if weight is not None:
        wt = weight.to(logp.dtype)[torch.where(valid, target, torch.zeros_like(target))]
        wt = torch.where(valid, wt, torch.zeros_like(wt))
    else:
        wt = valid.to(logp.dtype)
    elem = -picked * wt
    if reduction == "none":
        return elem.to(in_dtype)
    return reduce_scalar_loss(elem.sum(), wt.sum(), reduction, reduce_groups).to(in_dtype)


def distributed_cross_entropy(
    logits, target, *, weight=None, ignore_index: int = -100, reduction: str = "mean", label_smoothing: float = 0.0,
    dim: int = 1, channel_group=None, reduce_groups=None,
) -> torch.Tensor:
    """``F.cross_entropy`` on logits whose class dimension ``dim`` is split over
    ``channel_group``.  Targets are class indices (supports ``weight``, ``ignore_index``,
    ``label_smoothing``, also together, with torch's rule for the combination) or class probabilities
    sharded like the logits (none of the three options)."""
    _check_reduction(reduction)
    dim = dim % logits.dim()
    in_dtype = logits.dtype
    if logits.is_cuda and not target.is_floating_point() and weight is None and label_smoothing == 0.0:
        from ...ops import loss_fused

        elem = loss_fused.maybe_fused_cross_entropy(logits, target, dim, channel_group, ignore_index)
        if elem is not None:
            if reduction == "none":
                return elem.to(in_dtype)
            wt = (target != ignore_index).to(torch.float32)
            return reduce_scalar_loss(elem.sum(), wt.sum(), reduction, reduce_groups).to(in_dtype)
    with torch.autocast(logits.device.type, enabled=False):
        scores = logits.to(torch.promote_types(in_dtype, torch.float32))
        logp = distributed_log_softmax(scores, dim, channel_group)
        if target.is_floating_point():
            if weight is not None or label_smoothing != 0.0 or ignore_index != -100:
                raise NotImplementedError(
                    "class-probability targets support neither weight, ignore_index nor label_smoothing"
                )
            elem = redundant_all_reduce(-(target.to(logp.dtype) * logp).sum(dim=dim), channel_group)
            if reduction == "none":
                return elem.to(in_dtype)
            count = torch.full((), float(elem.numel()), device=elem.device)
            return reduce_scalar_loss(elem.sum(), count, reduction, reduce_groups).to(in_dtype)
        picked, valid = _pick_target(logp, target, dim, channel_group, ignore_index)
        if label_smoothing != 0.0:
            c_local = logp.shape[dim]
            c_global = c_local * _gsize(channel_group)
            if weight is not None:           # torch's rule: both terms carry the class weights, the mean divides by sum w[y]
                wg = weight.to(logp.dtype)
                wt = torch.where(valid, wg[torch.where(valid, target, torch.zeros_like(target))], torch.zeros((), dtype=logp.dtype, device=logp.device))
                shape = [1] * logp.dim()
                shape[dim] = c_local
                w_local = wg[_grank(channel_group) * c_local:(_grank(channel_group) + 1) * c_local].view(shape)
                smooth = (logp * w_local).sum(dim=dim) * (label_smoothing / c_global)
                picked = picked * wt
            else:
                wt = valid.to(logp.dtype)
                smooth = logp.sum(dim=dim) * (label_smoothing / c_global)
            both = redundant_all_reduce(torch.stack((picked, smooth)), channel_group)
            elem = -((1.0 - label_smoothing) * both[0] + both[1])
            elem = torch.where(valid, elem, torch.zeros_like(elem))
        else:
            picked = redundant_all_reduce(picked, channel_group)
            if weight is not None:
                wt = weight.to(logp.dtype)[torch.where(valid, target, torch.zeros_like(target))]
                wt = torch.where(valid, wt, torch.zeros_like(wt))
            else:
                wt = valid.to(logp.dtype)
            elem = -picked * wt
        if reduction == "none":
            return elem.to(in_dtype)
        return reduce_scalar_loss(elem.sum(), wt.sum(), reduction, reduce_groups).to(in_dtype)
