"""``nn.Module`` front-ends of the distributed losses (no parameters).

Reference parity: jigsaw/modules/loss/_classification/loss.py:12-337,
_regression/loss.py:11-208.
"""

from __future__ import annotations

import torch

from ..._core.shard_repr import shard_repr
from . import _functional as LF


class _Loss(torch.nn.Module):
    def get_parameter_count(self) -> int:
        return 0

    def extra_repr(self) -> str:
        """Size of the class-sharding group (classification losses only), then of the reduction groups (one size
        per group if a sequence was given)."""
        fields = {"channel": self.channel_group} if hasattr(self, "channel_group") else {}
        return shard_repr(**fields, reduce_groups=getattr(self, "reduce_groups", None))


class DistributedNLLLoss(_Loss):
    """``torch.nn.NLLLoss`` for log-probabilities with a sharded class dimension."""

    def __init__(self, channel_group=None, reduce_groups=None, *, weight=None, ignore_index: int = -100,
                 reduction: str = "mean", dim: int = 1) -> None:
        super().__init__()
        self.channel_group, self.reduce_groups = channel_group, reduce_groups
        self.register_buffer("weight", weight)
        self.ignore_index, self.reduction, self.dim = ignore_index, reduction, dim

    def forward(self, log_probs: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
        return LF.distributed_nll_loss(
            log_probs, target, weight=self.weight, ignore_index=self.ignore_index, reduction=self.reduction,
            dim=self.dim, channel_group=self.channel_group, reduce_groups=self.reduce_groups,
        )


class DistributedCrossEntropyLoss(_Loss):
    """``torch.nn.CrossEntropyLoss`` for logits with a sharded class dimension."""

    def __init__(self, channel_group=None, reduce_groups=None, *, weight=None, ignore_index: int = -100,
                 reduction: str = "mean", label_smoothing: float = 0.0, dim: int = 1) -> None:
        super().__init__()
        self.channel_group, self.reduce_groups = channel_group, reduce_groups
        self.register_buffer("weight", weight)
        self.ignore_index, self.reduction = ignore_index, reduction
        self.label_smoothing, self.dim = label_smoothing, dim

    def forward(self, logits: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
        return LF.distributed_cross_entropy(
            logits, target, weight=self.weight, ignore_index=self.ignore_index, reduction=self.reduction,
            label_smoothing=self.label_smoothing, dim=self.dim, channel_group=self.channel_group,
            reduce_groups=self.reduce_groups,
        )


class DistributedBCELoss(_Loss):
    """``torch.nn.BCELoss`` on a sharded tensor; list every sharding group in ``reduce_groups``."""

    def __init__(self, reduce_groups=None, *, weight=None, reduction: str = "mean") -> None:
        super().__init__()
        self.reduce_groups, self.reduction = reduce_groups, reduction
        self.register_buffer("weight", weight)

    def forward(self, probs: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
        return LF.distributed_binary_cross_entropy(
            probs, target, weight=self.weight, reduction=self.reduction, reduce_groups=self.reduce_groups
        )


class DistributedBCEWithLogitsLoss(_Loss):
    """``torch.nn.BCEWithLogitsLoss`` on a sharded tensor."""

    def __init__(self, reduce_groups=None, *, weight=None, pos_weight=None, reduction: str = "mean") -> None:
        super().__init__()
        self.reduce_groups, self.reduction = reduce_groups, reduction
        self.register_buffer("weight", weight)
        self.register_buffer("pos_weight", pos_weight)

    def forward(self, logits: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
        return LF.distributed_binary_cross_entropy_with_logits(
            logits, target, weight=self.weight, pos_weight=self.pos_weight, reduction=self.reduction,
            reduce_groups=self.reduce_groups,
        )


class DistributedMSELoss(_Loss):
    """``torch.nn.MSELoss`` on a sharded tensor."""

    def __init__(self, reduce_groups=None, *, reduction: str = "mean") -> None:
        super().__init__()
        self.reduce_groups, self.reduction = reduce_groups, reduction

    def forward(self, input: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
        return LF.distributed_mse_loss(input, target, reduction=self.reduction, reduce_groups=self.reduce_groups)


class DistributedL1Loss(_Loss):
    """``torch.nn.L1Loss`` on a sharded tensor."""

    def __init__(self, reduce_groups=None, *, reduction: str = "mean") -> None:
        super().__init__()
        self.reduce_groups, self.reduction = reduce_groups, reduction

    def forward(self, input: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
        return LF.distributed_l1_loss(input, target, reduction=self.reduction, reduce_groups=self.reduce_groups)


class DistributedSmoothL1Loss(_Loss):
    """``torch.nn.SmoothL1Loss`` on a sharded tensor."""

    def __init__(self, reduce_groups=None, *, beta: float = 1.0, reduction: str = "mean") -> None:
        super().__init__()
        self.reduce_groups, self.reduction, self.beta = reduce_groups, reduction, beta

    def forward(self, input: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
        return LF.distributed_smooth_l1_loss(
            input, target, beta=self.beta, reduction=self.reduction, reduce_groups=self.reduce_groups
        )
