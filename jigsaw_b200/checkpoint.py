"""Checkpoints of sharded models: gather to a plain state dict, or save / load one file per
model shard with a manifest that lets a different mesh read it back.

Every distributed layer describes its own cut with ``shard_spec()`` (parameter name ->
``((dim, group), ...)``); everything else in a model is replicated.  From that:

``full_state_dict(model)``
    plain PyTorch state dict with the global tensors (collective: all-gathers over the groups
    that cut each parameter).  Keys are the usual dotted names, so a serial copy of the model
    or any later tool can read it without this package.
``load_full_state_dict(model, state)``
    the inverse: every rank keeps its block of each global tensor.  No communication.
``save_sharded(model, mesh, directory)`` / ``load_sharded(model, mesh, directory)``
    one file per distinct shard (ranks that hold copies - data-parallel replicas, tile ranks of
    a replicated weight - do not write) plus ``manifest.json`` with the mesh axis sizes and,
    per tensor, the global shape and which dimension is cut over which axis.  Loading works on
    any mesh whose cuts divide the global shapes: every rank reads just the blocks that
    overlap its own shard.  With ``optimizer=`` the optimizer's state travels too (moments cut
    like their parameters, counters and hyper-parameters in the manifest): resume on any mesh.

Reference parity: the reference has no checkpoint module; its documented recipe is "ranks with
dp rank 0 save one ``state_dict`` per model rank" (examples/ddp.py:20-22) and
``reshard_parameters`` / ``convert_to_torch`` per layer (examples/reshard.py:78-107).  This
module packages that recipe and adds the manifest so a checkpoint no longer depends on the
mesh that wrote it.
"""

from __future__ import annotations

import json
import os
from collections.abc import Mapping
from itertools import product
from pathlib import Path
from typing import Any

import torch
import torch.distributed as dist

from ._core.placement import gather_dim

Layout = dict[str, tuple[tuple[int, dist.ProcessGroup], ...]]
MANIFEST = "manifest.json"
FORMAT = 1


def parameter_layout(model: torch.nn.Module) -> Layout:
    """``{state-dict key: ((dim, group), ...)}`` for every entry of ``model.state_dict()``;
    replicated entries map to ``()``.  Cuts over size-1 groups are dropped."""
    layout: Layout = {k: () for k in model.state_dict().keys()}
    for prefix, module in model.named_modules():
        spec = getattr(module, "shard_spec", None)
        if spec is None:
            continue
        for name, cuts in spec().items():
            key = f"{prefix}.{name}" if prefix else name
            if key in layout:
                layout[key] = tuple((d, g) for d, g in cuts if g is not None and g.size() > 1)
    return layout


def row_orders(model: torch.nn.Module) -> dict[str, tuple[str, Any]]:
    """``{key: (tag, reorder)}`` for tensors whose row order depends on the mesh (the qkv
    projection of ``DistributedAttention``); ``reorder(tensor, from_tag, to_tag)`` converts."""
    out: dict[str, tuple[str, Any]] = {}
    for prefix, module in model.named_modules():
        tags = getattr(module, "row_order_tags", None)
        if tags is None:
            continue
        for name, tag in tags().items():
            out[f"{prefix}.{name}" if prefix else name] = (tag, module.reorder_rows)
    return out


def _serial_tag(tag: str) -> str:
    kind, _, *rest = tag.split(":")
    return ":".join((kind, "1", *rest))


def full_state_dict(model: torch.nn.Module, canonical: bool = True) -> dict[str, torch.Tensor]:
    """Global tensors of a sharded model (collective; every rank gets the full dict).

    With ``canonical`` (default) mesh-dependent row orders are undone, so the result is what
    the same model holds on a single rank."""
    layout = parameter_layout(model)
    orders = row_orders(model) if canonical else {}
    out: dict[str, torch.Tensor] = {}
    with torch.no_grad():
        for key, value in model.state_dict().items():
            for dim, group in layout[key]:
                value = gather_dim(value, group, dim)
            value = value.detach().clone()
            if key in orders:
                tag, reorder = orders[key]
                value = reorder(value, tag, _serial_tag(tag))
            out[key] = value
    return out


def load_full_state_dict(model: torch.nn.Module, state: Mapping[str, torch.Tensor], strict: bool = True,
                         canonical: bool = True) -> None:
    """Give every rank its block of the global tensors in ``state`` (no communication).
    ``canonical`` must match the flag the state was gathered with."""
    layout = parameter_layout(model)
    orders = row_orders(model) if canonical else {}
    own = model.state_dict()
    missing = [k for k in own if k not in state]
    extra = [k for k in state if k not in own]
    if strict and (missing or extra):
        raise KeyError(f"state dict mismatch: missing {missing}, unexpected {extra}")
    with torch.no_grad():
        for key, target in own.items():
            if key not in state:
                continue
            value = state[key]
            if key in orders:
                tag, reorder = orders[key]
                value = reorder(value, _serial_tag(tag), tag)
            for dim, group in layout[key]:
                if value.shape[dim] % group.size():
                    raise ValueError(f"{key}: dimension {dim} of size {value.shape[dim]} does not split {group.size()} ways")
                n = value.shape[dim] // group.size()
                value = value.narrow(dim, group.rank() * n, n)
            if tuple(value.shape) != tuple(target.shape):
                raise ValueError(f"{key}: block of shape {tuple(value.shape)} does not fit the local {tuple(target.shape)}")
            target.copy_(value.to(device=target.device, dtype=target.dtype))


# --------------------------------------------------------------------------- sharded files
def _axis_of(group: dist.ProcessGroup, mesh: Mapping[str, dist.ProcessGroup]) -> str:
    ranks = dist.get_process_group_ranks(group)
    for name, g in mesh.items():
        if g is group or dist.get_process_group_ranks(g) == ranks:
            return name
    raise ValueError(f"group over ranks {ranks} is not an axis of the mesh {list(mesh)}")


def _mesh_groups(mesh: Any) -> dict[str, dist.ProcessGroup]:
    """Plain ``{axis: group}`` of the real axes of ``mesh``.  Derived axes are not coordinates of a shard:
    a ``ProcessMesh`` lists its real axes (``axis_sizes``); in a plain ``{name: group}`` mapping (which may
    carry the flattened ``"model"`` group beside the axes it is made of) a group is derived when its
    ranks contain all ranks of another non-trivial group, and a second name for the same ranks is dropped."""
    sizes = getattr(mesh, "axis_sizes", None)
    if sizes:
        return {n: mesh[n] for n in sizes}
    ranks = {n: frozenset(dist.get_process_group_ranks(g)) for n, g in mesh.items()}
    real: dict[str, dist.ProcessGroup] = {}
    for n in sorted(mesh, key=lambda name: name == "model"):      # the flattened group's name loses against an axis name
        g = mesh[n]
        derived = any(m != n and len(ranks[m]) > 1 and ranks[m] < ranks[n] for m in mesh)
        repeated = any(ranks[m] == ranks[n] and len(ranks[n]) > 1 for m in real)
        if not derived and not repeated:
            real[n] = g
    return real


def _shard_file(coord: Mapping[str, int], stem: str = "shard") -> str:
    return stem + "".join(f"-{a}{i}" for a, i in sorted(coord.items())) + ".pt"


def _describe(state: Mapping[str, torch.Tensor], layout: Layout, orders: dict, groups: dict) -> tuple[dict, set]:
    """Manifest entries of ``state`` and the mesh axes that cut any of its tensors."""
    cut_axes: set[str] = set()
    entries: dict[str, dict] = {}
    for key, value in state.items():
        cuts = [(d, _axis_of(g, groups)) for d, g in layout[key]]
        if len({a for _, a in cuts}) != len(cuts):
            raise ValueError(f"{key}: a mesh axis cuts more than one dimension ({cuts}); such a layout cannot be stored")
        shape = list(value.shape)
        for d, axis in cuts:
            shape[d] *= groups[axis].size()
            cut_axes.add(axis)
        entries[key] = {"shape": shape, "dtype": str(value.dtype).removeprefix("torch."), "cuts": cuts}
        if key in orders:
            entries[key]["rows"] = orders[key][0]
    return entries, cut_axes


def _optimizer_tensors(model: torch.nn.Module, optimizer: torch.optim.Optimizer) -> tuple[dict[str, dict], dict[str, dict]]:
    """Optimizer state by parameter name: ``{state name: {parameter key: tensor}}`` for the entries
    shaped like their parameter (moments, momentum buffers), which are cut like the parameter, and
    ``{parameter key: {state name: number}}`` for the scalar entries (step counters)."""
    names = {id(p): key for key, p in model.named_parameters()}
    shaped: dict[str, dict] = {}
    scalars: dict[str, dict] = {}
    for p, st in optimizer.state.items():
        key = names.get(id(p))
        if key is None:
            continue
        for name, val in st.items():
            if torch.is_tensor(val) and val.dim() > 0 and val.shape == p.shape:
                shaped.setdefault(name, {})[key] = val
            elif torch.is_tensor(val) and val.numel() == 1:
                scalars.setdefault(key, {})[name] = float(val)
            elif isinstance(val, (int, float)):
                scalars.setdefault(key, {})[name] = val
    return shaped, scalars


def _group_settings(optimizer: torch.optim.Optimizer) -> list[dict]:
    """JSON-able hyper-parameters of every parameter group, and the device-side step counter that
    :class:`jigsaw_b200.optim.FusedAdam` keeps per group (``fused_step``)."""
    out = []
    for group in optimizer.param_groups:
        entry: dict[str, Any] = {}
        for k, v in group.items():
            if isinstance(k, str) and k != "params" and isinstance(v, (int, float, bool, str, list, tuple, type(None))):
                entry[k] = list(v) if isinstance(v, tuple) else v
            elif isinstance(k, str) and torch.is_tensor(v) and v.numel() == 1:
                entry[k] = float(v)                     # a device-side hyper-parameter (learning rate as a tensor)
            elif isinstance(k, tuple) and k and k[0] == "step" and torch.is_tensor(v):
                entry["fused_step"] = max(float(v), entry.get("fused_step", 0.0))
        out.append(entry)
    return out


def save_sharded(model: torch.nn.Module, mesh: Any, directory: str | os.PathLike, extra: dict | None = None,
                 optimizer: torch.optim.Optimizer | None = None) -> None:
    """Write this model's shards and the manifest into ``directory`` (collective).

    ``extra`` (JSON-serialisable: step counter, hyper-parameters ...) goes into the manifest.  With
    ``optimizer`` its state is written too: entries shaped like their parameter (Adam moments, momentum
    buffers) as shards cut like the parameter, scalar entries and the groups' hyper-parameters in the
    manifest, so that training resumes on any mesh (:func:`load_sharded` with the new optimizer).
    """
    groups = _mesh_groups(mesh)
    layout = parameter_layout(model)
    state = model.state_dict()
    orders = row_orders(model)
    entries, cut_axes = _describe(state, layout, orders, groups)
    shaped, scalars = _optimizer_tensors(model, optimizer) if optimizer is not None else ({}, {})
    directory = Path(directory)
    rank = dist.get_rank()
    if rank == 0:
        directory.mkdir(parents=True, exist_ok=True)
    dist.barrier()
    axes = sorted(cut_axes)
    # a rank writes iff it is the first copy: coordinate 0 on every axis that cuts nothing
    writer = all(g.rank() == 0 for a, g in groups.items() if a not in cut_axes)
    coord = {a: groups[a].rank() for a in axes}
    if writer:
        torch.save({k: v.detach().cpu() for k, v in state.items()}, directory / _shard_file(coord))
        for name, tensors in shaped.items():
            torch.save({k: v.detach().cpu() for k, v in tensors.items()}, directory / _shard_file(coord, f"optim-{name}"))
    if rank == 0:
        manifest = {
            "format": FORMAT,
            "axes": {a: groups[a].size() for a in groups},
            "shard_axes": axes,
            "tensors": entries,
            "extra": extra or {},
        }
        if optimizer is not None:
            manifest["optimizer"] = {
                "class": type(optimizer).__name__,
                "states": {name: _describe(tensors, layout, orders, groups)[0] for name, tensors in shaped.items()},
                "scalars": scalars,
                "groups": _group_settings(optimizer),
            }
        (directory / MANIFEST).write_text(json.dumps(manifest, indent=1))
    dist.barrier()


def load_sharded(model: torch.nn.Module, mesh: Any, directory: str | os.PathLike, strict: bool = True,
                 optimizer: torch.optim.Optimizer | None = None) -> dict:
    """Fill ``model`` (sharded over ``mesh``) from a checkpoint written on any mesh; returns the
    manifest's ``extra``.  Each rank reads only the files whose blocks overlap its shards.

    With ``optimizer`` (built over ``model.parameters()``) its state is restored from a checkpoint
    that was saved with one: moments are cut for this mesh like the parameters, step counters and the
    groups' hyper-parameters (learning rate included) come from the manifest."""
    directory = Path(directory)
    manifest = json.loads((directory / MANIFEST).read_text())
    if manifest.get("format") != FORMAT:
        raise ValueError(f"unknown checkpoint format {manifest.get('format')!r}")
    layout = parameter_layout(model)
    own = model.state_dict()
    tensors: dict[str, dict] = manifest["tensors"]
    missing = [k for k in own if k not in tensors]
    unexpected = [k for k in tensors if k not in own]
    if strict and (missing or unexpected):
        raise KeyError(f"checkpoint mismatch: missing {missing}, unexpected {unexpected}")
    orders = row_orders(model)
    _fill(own, tensors, layout, orders, manifest, directory, "shard")
    if optimizer is not None:
        saved = manifest.get("optimizer")
        if saved is None:
            raise KeyError("the checkpoint holds no optimizer state")
        _restore_optimizer(model, optimizer, saved, layout, orders, manifest, directory)
    return manifest.get("extra", {})


def _restore_optimizer(model: torch.nn.Module, optimizer: torch.optim.Optimizer, saved: dict, layout: Layout, orders: dict,
                       manifest: dict, directory: Path) -> None:
    params = dict(model.named_parameters())
    for name, entries in saved["states"].items():
        own = {}
        for key in entries:
            if key not in params:
                raise KeyError(f"optimizer state for unknown parameter {key}")
            st = optimizer.state[params[key]]
            if name not in st or not torch.is_tensor(st[name]) or st[name].shape != params[key].shape:
                st[name] = torch.zeros_like(params[key], memory_format=torch.preserve_format)
            own[key] = st[name]
        _fill(own, entries, layout, orders, manifest, directory, f"optim-{name}")
    fused = type(optimizer).__name__ == "FusedAdam"
    for key, values in saved["scalars"].items():
        if key not in params:
            continue
        st = optimizer.state[params[key]]
        for name, val in values.items():
            if torch.is_tensor(st.get(name)):
                st[name].fill_(val)
            elif fused or name != "step":
                st[name] = val
            else:                                   # PyTorch's optimizers keep their step counters as fp32 scalars
                st[name] = torch.tensor(float(val), dtype=torch.float32)
    for group, settings in zip(optimizer.param_groups, saved["groups"]):
        step = settings.get("fused_step")
        for k, v in settings.items():
            if k != "fused_step" and k in group:
                if torch.is_tensor(group[k]):
                    group[k].fill_(v)
                else:
                    group[k] = tuple(v) if isinstance(group[k], tuple) and isinstance(v, list) else v
        if step is not None:
            for p in group["params"]:
                if p.is_cuda:
                    group[("step", p.device)] = torch.full((), float(step), dtype=torch.float32, device=p.device)
                elif "exp_avg" in optimizer.state[p]:
                    optimizer.state[p].setdefault("step", int(step))


def _fill(own: Mapping[str, torch.Tensor], tensors: Mapping[str, dict], layout: Layout, orders: dict, manifest: dict,
          directory: Path, stem: str) -> None:
    """Copy into every tensor of ``own`` (this rank's blocks, cut as ``layout`` says) its part of the
    global tensors that the files ``<stem>-<coordinates>.pt`` hold in the source mesh's blocks."""
    src_sizes: dict[str, int] = manifest["axes"]
    src_axes: list[str] = manifest["shard_axes"]
    files: dict[str, dict] = {}

    def read(coord: dict[str, int]) -> dict:
        name = _shard_file(coord, stem)
        if name not in files:
            files[name] = torch.load(directory / name, map_location="cpu", weights_only=True)
        return files[name]

    def assemble(key: str, entry: dict) -> torch.Tensor:
        """The whole global tensor from every source block (used when rows must be reordered)."""
        shape = entry["shape"]
        src_cut = {axis: d for d, axis in entry["cuts"]}
        full = None
        for combo in product(*(range(src_sizes[a]) if a in src_cut else range(1) for a in src_axes)):
            coord = dict(zip(src_axes, combo))
            block = read(coord)[key]
            if full is None:
                full = torch.empty(shape, dtype=block.dtype)
            dst = full
            for axis, d in src_cut.items():
                n = shape[d] // src_sizes[axis]
                dst = dst.narrow(d, coord[axis] * n, n)
            dst.copy_(block)
        return full

    with torch.no_grad():
        for key, target in own.items():
            if key not in tensors:
                continue
            entry = tensors[key]
            shape = entry["shape"]
            if key in orders and entry.get("rows", orders[key][0]) != orders[key][0]:
                tag, reorder = orders[key]
                value = reorder(assemble(key, entry), entry["rows"], tag)
                for d, g in layout[key]:
                    n = value.shape[d] // g.size()
                    value = value.narrow(d, g.rank() * n, n)
                target.copy_(value.to(device=target.device, dtype=target.dtype))
                continue
            # my block in global coordinates
            lo = [0] * len(shape)
            hi = list(shape)
            for d, g in layout[key]:
                if shape[d] % g.size():
                    raise ValueError(f"{key}: dimension {d} of size {shape[d]} does not split {g.size()} ways")
                n = shape[d] // g.size()
                lo[d], hi[d] = g.rank() * n, (g.rank() + 1) * n
            if [h - low for low, h in zip(lo, hi)] != list(target.shape):
                raise ValueError(f"{key}: global shape {shape} gives a block that does not fit the local {tuple(target.shape)}")
            # source blocks that overlap it
            src_cut = {axis: d for d, axis in entry["cuts"]}
            ranges = []
            for axis in src_axes:
                if axis in src_cut:
                    d = src_cut[axis]
                    n = shape[d] // src_sizes[axis]
                    ranges.append(range(lo[d] // n, (hi[d] - 1) // n + 1))
                else:
                    ranges.append(range(1))          # any copy will do: take coordinate 0
            for combo in product(*ranges):
                coord = dict(zip(src_axes, combo))
                block = read(coord)[key]
                dst, src = target, block
                for axis, d in src_cut.items():
                    n = shape[d] // src_sizes[axis]
                    b_lo = coord[axis] * n
                    o_lo, o_hi = max(lo[d], b_lo), min(hi[d], b_lo + n)
                    dst = dst.narrow(d, o_lo - lo[d], o_hi - o_lo)
                    src = src.narrow(d, o_lo - b_lo, o_hi - o_lo)
                for d in range(len(shape)):
                    if d not in src_cut.values() and (lo[d], hi[d]) != (0, shape[d]):
                        src = src.narrow(d, lo[d], hi[d] - lo[d])
                dst.copy_(src.to(device=target.device, dtype=target.dtype))
