"""Replica marks, gradient synchronisation, DDP composition and gradient clipping.

Reference parity: jigsaw/parallel/__init__.py:24-37 (the twelve public names); ``no_grad_sync`` and
``reduce_replica_grads`` (gradient accumulation in the in-graph mode), ``OverlappedGradSync`` (bucketed reduction
under the backward pass for any module) and ``overlapped_sum_plan`` (for fused multi-layer operations that sum their
own gradients under their backward pass) have no counterpart there.
"""

from .._core.public import set_module
from ._clip import clip_grad_norm_
from ._ddp import check_ddp, wrap_ddp
from ._joint import JointCommHookState, joint_comm_hook, register_joint_comm_hook
from ._replicas import broadcast_replicas, mark_replicated, replica_groups
from ._sync import (OverlappedGradSync, no_grad_sync, overlapped_sum_plan, reduce_replica_grads, sync_grad, synced_call,
                    synced_parameters)

__all__ = [
    "JointCommHookState",
    "OverlappedGradSync",
    "broadcast_replicas",
    "check_ddp",
    "clip_grad_norm_",
    "joint_comm_hook",
    "mark_replicated",
    "no_grad_sync",
    "overlapped_sum_plan",
    "reduce_replica_grads",
    "register_joint_comm_hook",
    "replica_groups",
    "sync_grad",
    "synced_call",
    "synced_parameters",
    "wrap_ddp",
]

set_module(globals(), __all__)
