"""In-graph gradient synchronisation of replicated parameters.

``sync_grad(w, b)`` returns views whose backward sums the incoming gradients over the
replica groups of each marked parameter: one flat all-reduce per (groups, dtype) bucket
and group.  Under a DDP with the joint hook registered the sum is replaced by a scale
(the hook reduces).  The returned tensors carry no mark, so nested or re-entered
forwards never reduce twice.

Setting ``JIGSAW_DISABLE_GRAD_SYNC=1`` turns the function into a pass-through: a mutation
switch for tests that must *fail* when synchronisation is missing.

Reference parity: jigsaw/parallel/_sync.py:13-16 (switch), :19-53 (_SyncGrad), :56-83
(_ScaleGrad), :86-132 (sync_grad), :135-194 (synced_parameters / synced_call).
"""

from __future__ import annotations

import contextlib
import os
from collections.abc import Iterable, Iterator
from typing import Any

import torch
import torch.distributed as dist

from ._ddp import check_active_ddp
from ._joint import JointCommHookState, active_joint_state, joint_state_of
from ._replicas import Groups, merged_group, replica_groups, replica_rank_set

_SYNC_DISABLED = os.environ.get("JIGSAW_DISABLE_GRAD_SYNC", "") == "1"
_deferred = 0          # nesting depth of no_grad_sync()


def _all_reduce_sum(flat: torch.Tensor, group: dist.ProcessGroup) -> None:
    if flat.is_cuda and group.size() > 1:
        from ..ops import reduce_fused

        # one own kernel over peer memory (bit-identical on every rank) instead of the library collective
        if reduce_fused.maybe_fused_all_reduce([flat], dist.get_process_group_ranks(group)):
            return
    dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)


def _reduce_flat(flat: torch.Tensor, groups: Groups) -> None:
    if flat.is_cuda and len(groups) > 1:
        from ..ops import reduce_fused

        # all axes in one launch: the kernel addresses the copies by rank, it needs no process group
        ranks = replica_rank_set(groups)
        if len(ranks) <= 8 and reduce_fused.usable([flat], ranks) and reduce_fused.maybe_fused_all_reduce([flat], ranks):
            return
    whole = merged_group(groups)
    if whole is not None:
        _all_reduce_sum(flat, whole)
        return
    for g in groups:
        _all_reduce_sum(flat, g)


class _SumGradOverGroups(torch.autograd.Function):
    """Identity forward; backward = SUM all-reduce of all gradients, flattened together."""

    @staticmethod
    def forward(groups: Groups, *tensors: torch.Tensor) -> tuple[torch.Tensor, ...]:
        return tuple(t.view_as(t) for t in tensors)

    @staticmethod
    def setup_context(ctx: Any, inputs: tuple, output: tuple) -> None:
        ctx.groups = inputs[0]

    @staticmethod
    def backward(ctx: Any, *grads: torch.Tensor) -> tuple:
        if len(grads) == 1:
            flat = grads[0].contiguous().clone().view(-1)
        else:
            flat = torch.cat([g.reshape(-1) for g in grads])
        _reduce_flat(flat, ctx.groups)
        outs, offset = [], 0
        for g in grads:
            outs.append(flat[offset : offset + g.numel()].view_as(g))
            offset += g.numel()
        return (None, *outs)

    @staticmethod
    def vmap(info: Any, in_dims: tuple, groups: Groups, *tensors: Any) -> tuple:
        # elementwise in the batch: reduce the stacked members in one go
        return _SumGradOverGroups.apply(groups, *tensors), tuple(in_dims[1:])


class _ScaleGrad(torch.autograd.Function):
    """Identity forward; backward multiplies by ``factor`` (the joint hook does the sum)."""

    @staticmethod
    def forward(factor: float, *tensors: torch.Tensor) -> tuple[torch.Tensor, ...]:
        return tuple(t.view_as(t) for t in tensors)

    @staticmethod
    def setup_context(ctx: Any, inputs: tuple, output: tuple) -> None:
        ctx.factor = inputs[0]

    @staticmethod
    def backward(ctx: Any, *grads: torch.Tensor) -> tuple:
        return (None, *(g * ctx.factor for g in grads))

    @staticmethod
    def vmap(info: Any, in_dims: tuple, factor: float, *tensors: Any) -> tuple:
        return _ScaleGrad.apply(factor, *tensors), tuple(in_dims[1:])


def sync_grad(*tensors: torch.Tensor | None) -> tuple[torch.Tensor | None, ...]:
    """Route marked parameters through the in-graph gradient sum (or scale, see module doc).

    Unmarked tensors, ``None``, tensors that do not require grad and everything under
    ``torch.no_grad()`` pass through untouched.
    """
    result = list(tensors)
    if not dist.is_initialized():        # a single process: nothing is replicated
        return tuple(result)
    check_active_ddp()
    if _SYNC_DISABLED or not torch.is_grad_enabled():
        return tuple(result)
    joint = active_joint_state()
    buckets: dict[tuple[Groups, torch.dtype, JointCommHookState | None], list[int]] = {}
    for i, t in enumerate(tensors):
        if t is None or not t.requires_grad:
            continue
        groups = replica_groups(t)
        if not groups:
            continue
        buckets.setdefault((groups, t.dtype, joint_state_of(t, joint)), []).append(i)
    for (groups, _, state), idx in buckets.items():
        members = [tensors[i] for i in idx]
        if state is None:
            if _deferred:
                continue                     # gradient accumulation: reduce_replica_grads() sums once at the end
            routed = _SumGradOverGroups.apply(groups, *members)
        else:
            routed = _ScaleGrad.apply(state.factor(groups), *members)
        for i, r in zip(idx, routed):
            result[i] = r
    return tuple(result)


def overlapped_sum_plan(tensors: Iterable[torch.Tensor | None]) -> list[int] | None:
    """For fused multi-layer operations that produce the gradients of several replicated parameters one
    after another: the world ranks over which ALL of ``tensors`` must be summed, when that sum may be
    started per layer on a side stream while the operation's backward pass continues (CUDA, one common
    set of replica groups, at most eight copies, no gradient accumulation in progress, no DDP joint hook
    in charge).  ``None`` means: route the parameters through :func:`sync_grad` instead."""
    if not dist.is_initialized() or _SYNC_DISABLED or _deferred or not torch.is_grad_enabled():
        return None
    if active_joint_state() is not None:
        return None
    common = None
    for t in tensors:
        if t is None or not t.requires_grad:
            continue
        if not t.is_cuda or t.dtype != torch.float32:
            return None
        groups = replica_groups(t)
        key = tuple(sorted(tuple(dist.get_process_group_ranks(g)) for g in groups))
        if common is None:
            common = (key, groups)
        elif common[0] != key:
            return None
    if common is None or not common[1]:
        return None
    ranks = replica_rank_set(common[1])
    return ranks if 2 <= len(ranks) <= 8 else None


@contextlib.contextmanager
def no_grad_sync() -> Iterator[None]:
    """Gradient accumulation without a reduction per micro-batch: inside the block :func:`sync_grad`
    leaves the gradients of replicated parameters local (every rank accumulates its own contribution
    in ``.grad``); call :func:`reduce_replica_grads` once after the last micro-batch.  The counterpart
    of DDP's ``no_sync`` for the in-graph mode; under the joint DDP hook, where DDP reduces, it changes
    nothing.

        with jb.parallel.no_grad_sync():
            for micro in batches:
                loss_fn(model(micro.x), micro.y).backward()
        jb.parallel.reduce_replica_grads(model)
        optimizer.step()
    """
    global _deferred
    _deferred += 1
    try:
        yield
    finally:
        _deferred -= 1


def reduce_replica_grads(module_or_parameters: torch.nn.Module | Iterable[torch.Tensor]) -> None:
    """SUM all-reduce the accumulated ``.grad`` of every marked parameter over its replica groups:
    one flattened all-reduce per (groups, dtype) bucket (collective; the same call on every rank)."""
    if not dist.is_initialized() or _SYNC_DISABLED:
        return
    params = module_or_parameters.parameters() if isinstance(module_or_parameters, torch.nn.Module) else module_or_parameters
    buckets: dict[tuple[Groups, torch.dtype], list[torch.Tensor]] = {}
    for p in params:
        groups = replica_groups(p)
        if p.grad is None or not groups:
            continue
        buckets.setdefault((groups, p.grad.dtype), []).append(p.grad)
    with torch.no_grad():
        for (groups, _), grads in buckets.items():
            flat = torch.cat([g.reshape(-1) for g in grads])
            _reduce_flat(flat, groups)
            offset = 0
            for g in grads:
                g.copy_(flat[offset: offset + g.numel()].view_as(g))
                offset += g.numel()


def synced_parameters(module: torch.nn.Module) -> dict[str, torch.Tensor]:
    """``{name: synced tensor}`` for the marked parameters of ``module`` (empty when none,
    or when grad mode is off), for ``torch.func.functional_call``."""
    marked = {n: p for n, p in module.named_parameters() if replica_groups(p)}
    if not marked:
        return {}
    routed = sync_grad(*marked.values())
    return {n: r for (n, p), r in zip(marked.items(), routed) if r is not None and r is not p}


def synced_call(module: torch.nn.Module, *args: Any, **kwargs: Any) -> Any:
    """Call a foreign ``module`` (e.g. a plain ``nn.LayerNorm`` whose parameters were marked
    by hand) with its marked parameters routed through :func:`sync_grad`."""
    routed = synced_parameters(module)
    if not routed:
        return module(*args, **kwargs)
    return torch.func.functional_call(module, routed, args, kwargs)


class OverlappedGradSync:
    """Sum the gradients of replicated parameters bucket by bucket WHILE the backward pass is still running.

    The in-graph mode (:func:`sync_grad`) reduces inside the autograd graph, on the stream of the backward
    pass: every reduction is on the critical path.  Inside this context the in-graph reduction is switched off
    (as under :func:`no_grad_sync`); instead a hook fires when a marked parameter's gradient has been
    accumulated, parameters are collected into buckets of about ``bucket_bytes`` per (replica groups, dtype),
    and a full bucket is reduced at once:

    * CUDA, fp32, at most eight copies: the peer-memory all-reduce kernel on a side stream
      (:class:`jigsaw_b200.ops.reduce_fused.OverlappedReducer`), in place, bit-identical on every rank, while the
      remaining gradient kernels keep the GPU busy;
    * otherwise: an asynchronous ``all_reduce`` of the flattened bucket per group, copied back at the end.

    Leaving the context (or :meth:`finish`) flushes the partial buckets and waits; the optimizer step follows.

        with jb.parallel.OverlappedGradSync(model):
            loss_fn(model(x), y).backward()
        optimizer.step()

    One backward pass per context: the hooks reduce what is in ``.grad`` when they fire, so for gradient
    accumulation wrap only the LAST micro-batch (the earlier ones under :func:`no_grad_sync`).  Every rank must
    run the same model, so that the hooks fire in the same order everywhere (the assumption DDP's buckets make).
    Under the joint DDP hook, where DDP reduces, the context changes nothing.

    Reference parity: the per-module blocking reduction of jigsaw/parallel/_sync.py:19-53 and the bucket hook of
    jigsaw/parallel/_joint.py:215-279; the overlap outside DDP has no counterpart there.
    """

    def __init__(self, module_or_parameters: torch.nn.Module | Iterable[torch.Tensor], bucket_bytes: int = 1 << 20) -> None:
        params = module_or_parameters.parameters() if isinstance(module_or_parameters, torch.nn.Module) else module_or_parameters
        self.params = [p for p in params if p.requires_grad and replica_groups(p)]
        self.bucket_bytes = int(bucket_bytes)
        self._handles: list[Any] = []
        self._buckets: dict[tuple, list[torch.Tensor]] = {}
        self._pending: list[tuple] = []            # (flat, grads, works) of the library path
        self._reducers: dict[tuple, Any] = {}
        self.launched = 0                          # buckets reduced so far (for tests and logs)
        self._active = False

    # ------------------------------------------------------------------ context
    def __enter__(self) -> "OverlappedGradSync":
        global _deferred
        if self._active:
            raise RuntimeError("OverlappedGradSync is not re-entrant")
        self._active = True
        self._live = dist.is_initialized() and not _SYNC_DISABLED and active_joint_state() is None
        _deferred += 1
        if self._live:
            for p in self.params:
                self._handles.append(p.register_post_accumulate_grad_hook(self._on_grad))
        return self

    def __exit__(self, exc_type: Any, exc: Any, tb: Any) -> None:
        global _deferred
        try:
            if exc_type is None:
                self.finish()
        finally:
            for h in self._handles:
                h.remove()
            self._handles.clear()
            self._buckets.clear()
            _deferred -= 1
            self._active = False

    # ------------------------------------------------------------------ hooks
    def _on_grad(self, p: torch.Tensor) -> None:
        if p.grad is None:
            return
        groups = replica_groups(p)
        key = (groups, p.grad.dtype, p.grad.device)
        bucket = self._buckets.setdefault(key, [])
        bucket.append(p.grad)
        if sum(g.numel() * g.element_size() for g in bucket) >= self.bucket_bytes:
            self._reduce(key, self._buckets.pop(key))

    def _reduce(self, key: tuple, grads: list[torch.Tensor]) -> None:
        groups, dtype, device = key
        self.launched += 1
        if device.type == "cuda" and dtype == torch.float32:
            from ..ops import reduce_fused

            ranks = replica_rank_set(groups)
            if len(ranks) <= 8 and reduce_fused.usable(grads, ranks) and all(g.is_contiguous() for g in grads):
                red = self._reducers.get(tuple(ranks))
                if red is None:
                    red = self._reducers[tuple(ranks)] = reduce_fused.OverlappedReducer(device, ranks)
                red.add(grads)                      # in place, on the side stream
                return
        with torch.no_grad():
            flat = torch.cat([g.reshape(-1) for g in grads])
            whole = merged_group(groups)
            works = [dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=g, async_op=True) for g in ((whole,) if whole is not None else groups[:1])]
            self._pending.append((flat, grads, works, () if whole is not None else groups[1:]))

    def finish(self) -> None:
        """Reduce the partial buckets and wait for everything that is in flight (collective)."""
        for key in list(self._buckets):
            self._reduce(key, self._buckets.pop(key))
        for red in self._reducers.values():
            red.finish()
        with torch.no_grad():
            for flat, grads, works, later in self._pending:
                for w in works:
                    w.wait()
                for g in later:                     # further axes of a parameter replicated over several groups
                    dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=g)
                offset = 0
                for g in grads:
                    g.copy_(flat[offset: offset + g.numel()].view_as(g))
                    offset += g.numel()
        self._pending.clear()
