"""Replica marks: which process groups hold identical copies of a parameter.

A parameter that every rank of a group holds in full (a convolution weight over the
spatial axes, a bias over the token axis) sees only its rank's share of the gradient.
The mark records those groups on the parameter; :func:`sync_grad` sums the gradient over
them, :func:`clip_grad_norm_` and :func:`count_parameters` count such copies once, and
the DDP joint hook folds them into the data-parallel reduction.

Reference parity: jigsaw/parallel/_replicas.py:23-85 (mark), :88-101 (lookup), :104-147
(coalesced broadcast), :150-192 (divergence in float64, NaN-aware).
"""

from __future__ import annotations

from collections.abc import Iterable, Sequence

import torch
import torch.distributed as dist

MARK_ATTR = "_jigsaw_replica_groups"
Groups = tuple[dist.ProcessGroup, ...]


# A set of orthogonal axis groups that together tile one bigger group (the axes of a model
# replica and its flattened ``model`` group) can be reduced in one collective over that group.
_MERGED: dict[frozenset, "dist.ProcessGroup"] = {}


def register_merged_group(parts: "Sequence[dist.ProcessGroup]", whole: "dist.ProcessGroup") -> None:
    """Record that SUM over every group of ``parts`` in turn equals SUM over ``whole``."""
    live = [g for g in parts if g is not None and g.size() > 1]
    if len(live) < 2:
        return
    n = 1
    for g in live:
        n *= g.size()
    if n != whole.size():
        return
    _MERGED[frozenset(tuple(dist.get_process_group_ranks(g)) for g in live)] = whole


def merged_group(groups: "Sequence[dist.ProcessGroup]") -> "dist.ProcessGroup | None":
    if len(groups) < 2 or not _MERGED:
        return None
    return _MERGED.get(frozenset(tuple(dist.get_process_group_ranks(g)) for g in groups))


def replica_rank_set(groups: "Sequence[dist.ProcessGroup]") -> list[int]:
    """World ranks that hold a copy of a parameter replicated over ``groups`` (orthogonal axes of a
    regular mesh: the offsets along the axes add up), this rank included, sorted."""
    ranks = {dist.get_rank()}
    for g in groups:
        members = dist.get_process_group_ranks(g)
        mine = members[g.rank()]
        ranks = {r + (m - mine) for r in ranks for m in members}
    return sorted(ranks)


def _real_groups(groups: "dist.ProcessGroup | Iterable[dist.ProcessGroup | None] | None") -> Groups:
    if groups is None:
        return ()
    seq = [groups] if isinstance(groups, dist.ProcessGroup) else list(groups)
    return tuple(g for g in seq if g is not None and g.size() > 1)


def replica_groups(param: torch.Tensor | None) -> Groups:
    """Groups ``param`` is marked replicated over (``()`` when unmarked or ``None``)."""
    return getattr(param, MARK_ATTR, ())


def mark_replicated(
    param: torch.nn.Parameter,
    groups: "dist.ProcessGroup | Sequence[dist.ProcessGroup | None]",
    extend: bool = False,
) -> None:
    """Record that ``param`` is replicated over ``groups`` (size-1 groups and ``None`` are dropped).

    A second mark raises ``RuntimeError`` unless ``extend`` is true (its gradient would be
    summed twice); with ``extend`` the new groups are added and groups over an already
    marked rank set are skipped.  A group that meets the already marked ones in any rank
    besides the caller raises ``ValueError``: replica groups must be orthogonal mesh axes.
    """
    current = replica_groups(param)
    if current and not extend:
        raise RuntimeError(
            "parameter is already marked replicated; a second mark would sum its gradient twice. "
            "Pass extend=True to add groups to the mark."
        )
    wanted = _real_groups(groups)
    if not wanted:                       # nothing to add (also: a single process without a process group)
        return
    me = dist.get_rank()
    known = {tuple(dist.get_process_group_ranks(g)) for g in current}
    covered = {r for ranks in known for r in ranks}
    merged = list(current)
    for g in wanted:
        ranks = tuple(dist.get_process_group_ranks(g))
        if ranks in known:
            continue
        clash = (set(ranks) & covered) - {me}
        if clash:
            raise ValueError(
                f"group {list(ranks)} overlaps a replica group of this parameter in ranks "
                f"{sorted(clash)} besides rank {me}; replica groups must meet only in the calling "
                "rank, e.g. orthogonal mesh axes."
            )
        known.add(ranks)
        covered.update(ranks)
        merged.append(g)
    if merged:
        setattr(param, MARK_ATTR, tuple(merged))


def _coalesced_broadcast(params: list[torch.Tensor], group: dist.ProcessGroup, src: int) -> None:
    by_dtype: dict[torch.dtype, list[torch.Tensor]] = {}
    for p in params:
        by_dtype.setdefault(p.dtype, []).append(p)
    for plist in by_dtype.values():
        flat = torch.cat([p.detach().reshape(-1) for p in plist])
        dist.broadcast(flat, group_src=src, group=group)
        offset = 0
        for p in plist:
            n = p.numel()
            p.detach().copy_(flat[offset : offset + n].view_as(p))
            offset += n


def broadcast_replicas(module: torch.nn.Module, src: int = 0) -> None:
    """Collective: make every marked parameter equal to the copy on group rank ``src``.

    Broadcasting over each replica group in turn equalises the whole product of groups.
    One flat collective per (group tuple, group, dtype).
    """
    buckets: dict[Groups, list[torch.Tensor]] = {}
    for p in module.parameters():
        g = replica_groups(p)
        if g:
            buckets.setdefault(g, []).append(p)
    with torch.no_grad():
        for groups, params in buckets.items():
            for group in groups:
                _coalesced_broadcast(params, group, src)


def replica_divergence(
    params: Sequence[tuple[torch.Tensor, Sequence[dist.ProcessGroup | None]]],
) -> torch.Tensor:
    """``max |p - p_rank0|`` per parameter over each of its groups, as float64 (local result).

    NaN on both sides counts as equal; NaN on one side only gives ``inf``.  Collective
    over every listed group, in order.
    """
    device = params[0][0].device if params else torch.device("cpu")
    out = torch.zeros(len(params), dtype=torch.float64, device=device)
    buckets: dict[Groups, list[int]] = {}
    for i, (_, groups) in enumerate(params):
        key = _real_groups(groups)
        if key:
            buckets.setdefault(key, []).append(i)
    with torch.no_grad():
        for groups, idx in buckets.items():
            mine = torch.cat([params[i][0].detach().reshape(-1).to(torch.float64) for i in idx])
            sizes = [params[i][0].numel() for i in idx]
            for group in groups:
                ref = mine.clone()
                dist.broadcast(ref, group_src=0, group=group)
                diff = (mine - ref).abs().nan_to_num(nan=0.0)
                diff = torch.where(mine.isnan() != ref.isnan(), torch.full_like(diff, torch.inf), diff)
                offset = 0
                for i, n in zip(idx, sizes):
                    if n:
                        out[i] = torch.maximum(out[i], diff[offset : offset + n].max())
                    offset += n
    return out
