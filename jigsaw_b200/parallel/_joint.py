"""Joint gradient reduction of replicated parameters inside DDP's buckets.

For a parameter replicated over groups ``R`` the gradient must become
``AVG_dp(SUM_R(local))``.  Instead of a blocking sum over ``R`` in the backward pass plus
DDP's average over ``dp``, the joint hook averages once over the *joint group* (every rank
holding a copy: the component of this rank in the graph whose edges are ``dp`` and the
groups of ``R``) while :func:`sync_grad` merely scales the local gradient by
``|joint| / |dp|``.  One collective, overlapped with backward like any DDP bucket.

Joint groups are found with a union-find over the rank lists every rank contributes
(one ``all_gather_object`` over the default group), and cached per partition.

Reference parity: jigsaw/parallel/_joint.py:24-167 (state), :170-212 (partition by label
propagation), :215-279 (bucket hook), :282-296 (python-reducer path), :299-337 (register),
:340-404 (lookup helpers).
"""

from __future__ import annotations

from collections.abc import Callable
from typing import Any

import torch
import torch.distributed as dist
from torch.nn.parallel import DistributedDataParallel

from ._replicas import Groups, replica_groups

STATE_ATTR = "_jigsaw_joint_state"
PARAM_STATE_ATTR = "_jigsaw_joint_param_state"
_partition_cache: dict[tuple, dist.ProcessGroup] = {}


def _components(world: int, edges: list[list[int]]) -> list[list[int]]:
    """Connected components of ranks ``0..world-1`` joined by the given rank lists."""
    parent = list(range(world))

    def find(x: int) -> int:
        while parent[x] != x:
            parent[x] = parent[parent[x]]
            x = parent[x]
        return x

    for ranks in edges:
        for r in ranks[1:]:
            a, b = find(ranks[0]), find(r)
            if a != b:
                parent[max(a, b)] = min(a, b)
    comps: dict[int, list[int]] = {}
    for r in range(world):
        comps.setdefault(find(r), []).append(r)
    return [comps[k] for k in sorted(comps)]


def _group_for_partition(partition: list[list[int]]) -> dist.ProcessGroup:
    """This rank's group in ``partition``; created collectively on first use."""
    if len(partition) == 1:
        return dist.group.WORLD  # type: ignore[return-value]
    key = tuple(tuple(p) for p in partition)
    if key not in _partition_cache:
        group, _ = dist.new_subgroups_by_enumeration(partition)
        _partition_cache[key] = group
    return _partition_cache[key]


class JointCommHookState:
    """Per-DDP state: joint group and scale factor for every replica-group tuple.

    Construction is collective over the default group and must happen on every rank with
    an identically built model; ranks that disagree on the number of distinct
    replica-group tuples raise ``RuntimeError`` together.
    """

    def __init__(self, ddp: DistributedDataParallel) -> None:
        self.ddp = ddp
        self.dp: dist.ProcessGroup = ddp.process_group
        self.python_reducer: bool = bool(getattr(ddp, "_use_python_reducer", False))
        ignored: set[str] = set(getattr(ddp, "parameters_to_ignore", set()))
        reduced = [p for n, p in ddp.module.named_parameters() if n not in ignored and p.requires_grad]
        tuples: list[Groups] = []
        for p in reduced:
            r = replica_groups(p)
            if r and r not in tuples:
                tuples.append(r)
        world = dist.get_world_size()
        mine = {
            "n": len(tuples),
            "dp": sorted(dist.get_process_group_ranks(self.dp)),
            "rep": [[sorted(dist.get_process_group_ranks(g)) for g in r] for r in tuples],
        }
        everyone: list[Any] = [None] * world
        dist.all_gather_object(everyone, mine)
        if len({e["n"] for e in everyone}) != 1:
            raise RuntimeError(
                "ranks disagree on the number of distinct replica-group tuples; the jigsaw model "
                "must be built the same way on every rank"
            )
        self._group: dict[Groups, dist.ProcessGroup] = {}
        self._factor: dict[Groups, float] = {}
        for k, r in enumerate(tuples):
            edges = [e["dp"] for e in everyone]
            for e in everyone:
                edges.extend(e["rep"][k])
            group = _group_for_partition(_components(world, edges))
            self._group[r] = group
            self._factor[r] = group.size() / self.dp.size()
        self._of: dict[int, dist.ProcessGroup] = {
            id(p): self._group.get(replica_groups(p), self.dp) for p in reduced
        }
        setattr(ddp, STATE_ATTR, self)
        if self.python_reducer:
            for p in reduced:
                setattr(p, PARAM_STATE_ATTR, self)

    def reduces(self, param: torch.Tensor) -> bool:
        """Whether DDP's buckets (hence the hook) reduce ``param``."""
        return id(param) in self._of

    def factor(self, groups: Groups) -> float:
        """``|joint group| / |dp|`` for the replica-group tuple ``groups``."""
        return self._factor[groups]

    def group_of(self, param: torch.Tensor) -> dist.ProcessGroup:
        """Group over which the hook averages the gradient of ``param``."""
        return self._of[id(param)]


def joint_comm_hook(state: JointCommHookState, bucket: Any) -> "torch.futures.Future[torch.Tensor]":
    """DDP comm hook: average every gradient of the bucket over its parameter's joint group.

    Consecutive parameters with the same joint group form one run and one asynchronous
    all-reduce (pre-divided by the group size).  Under DDP's python reducer the hook is
    called with ``(grad, param)`` and reduces in place.
    """
    if isinstance(bucket, tuple):
        grad, param = bucket
        group = state.group_of(param)
        scaled = grad / group.size()
        dist.all_reduce(scaled, group=group)
        grad.copy_(scaled)
        return None  # type: ignore[return-value]
    flat = bucket.buffer()
    runs: list[list[Any]] = []
    offset = 0
    for p in bucket.parameters():
        g = state.group_of(p)
        if runs and runs[-1][0] is g:
            runs[-1][2] = offset + p.numel()
        else:
            runs.append([g, offset, offset + p.numel()])
        offset += p.numel()
    if offset != flat.numel():
        raise RuntimeError(f"bucket buffer has {flat.numel()} elements but its parameters {offset}")
    works = []
    for g, lo, hi in runs:
        piece = flat[lo:hi]
        piece.div_(g.size())
        works.append(dist.all_reduce(piece, group=g, async_op=True))

    def done(_: Any) -> torch.Tensor:
        for w in works[:-1]:
            w.get_future().wait()
        return flat

    return works[-1].get_future().then(done)


# DDP validates the hook's annotations as objects, not strings.
joint_comm_hook.__annotations__ = {
    "state": JointCommHookState,
    "bucket": dist.GradBucket,
    "return": torch.futures.Future[torch.Tensor],
}


def register_joint_comm_hook(
    ddp: DistributedDataParallel, wrapper: Callable[[Callable], Callable] | None = None
) -> JointCommHookState:
    """Collective (every rank, before the first forward): build the state and register the hook.

    ``wrapper`` may be a compression wrapper such as ``fp16_compress_wrapper``; it is
    rejected (``ValueError``) with DDP's python reducer, which has no buckets.
    """
    if wrapper is not None and getattr(ddp, "_use_python_reducer", False):
        raise ValueError(
            "comm hook wrappers need DDP's gradient buckets, which DDP's Python reducer "
            "(compiled autograd) does not have"
        )
    state = JointCommHookState(ddp)
    ddp.register_comm_hook(state, joint_comm_hook if wrapper is None else wrapper(joint_comm_hook))
    return state


def _hook_registered(state: JointCommHookState) -> bool:
    return any(s is state for _, s in getattr(state.ddp, "_comm_hooks", ()))


def _require_hook(state: JointCommHookState) -> None:
    if not _hook_registered(state):
        raise RuntimeError(
            "a JointCommHookState was built for this DDP but joint_comm_hook is not registered on "
            "it; without the hook the replicated gradients are never summed. Use "
            "jigsaw_b200.parallel.register_joint_comm_hook(ddp)."
        )


def active_joint_state() -> JointCommHookState | None:
    """Joint state of the DDP whose forward is currently running, if it has one."""
    ddp = getattr(DistributedDataParallel, "_active_ddp_module", None)
    state = getattr(ddp, STATE_ATTR, None) if ddp is not None else None
    if not isinstance(state, JointCommHookState):
        return None
    _require_hook(state)
    return state


def joint_state_of(param: torch.Tensor, active: JointCommHookState | None) -> JointCommHookState | None:
    """State whose hook will reduce ``param``: ``active`` if it reduces it, else the
    state pinned on the parameter (python reducer), else ``None``."""
    if active is not None:
        return active if active.reduces(param) else None
    state = getattr(param, PARAM_STATE_ATTR, None)
    if state is not None:
        _require_hook(state)
    return state
