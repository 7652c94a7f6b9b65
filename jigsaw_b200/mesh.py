"""Process mesh: named, ordered axes -> one process group per axis plus a ``model`` group.

The trailing axes are the model-parallel axes (one model replica spans them); leading
axes hold data-parallel copies.  Besides the groups, a :class:`ProcessMesh` records the
axis sizes and this rank's coordinate, which the placement model and the peer-memory
runtime use for index math instead of creating more communicators.

Reference parity: jigsaw/mesh.py:21-47 (ProcessMesh), :60-104 (size / model-axis
resolution), :107-191 (make_process_mesh).
"""

from __future__ import annotations

import math
from collections.abc import Mapping, Sequence

import torch
import torch.distributed as dist

from ._core.comm import check_backend

__all__ = ["ProcessMesh", "make_process_mesh"]


class ProcessMesh(dict):
    """``dict`` of axis name -> process group that also carries the n-d ``DeviceMesh``.

    Attributes
    ----------
    device_mesh : torch.distributed.device_mesh.DeviceMesh
        The named n-d mesh the axis groups were cut from (the ``model`` group is not a
        dimension of it), e.g. for ``DistributedDataParallel(device_mesh=mesh.device_mesh["dp"])``.
    axis_sizes : dict[str, int]
        Size of every named axis, slowest-varying first.
    model_axes : tuple[str, ...]
        The trailing axes spanned by the ``model`` group.
    """

    device_mesh: "dist.device_mesh.DeviceMesh"

    def __init__(
        self,
        groups: Mapping[str, dist.ProcessGroup],
        device_mesh: "dist.device_mesh.DeviceMesh",
        axis_sizes: Mapping[str, int] | None = None,
        model_axes: Sequence[str] | None = None,
    ) -> None:
        super().__init__(groups)
        self.device_mesh = device_mesh
        self.axis_sizes = dict(axis_sizes) if axis_sizes is not None else {k: g.size() for k, g in groups.items()}
        self.model_axes = tuple(model_axes) if model_axes is not None else tuple(self.axis_sizes)

    def coordinate(self) -> dict[str, int]:
        """This rank's index along every named axis."""
        return {name: self[name].rank() for name in self.axis_sizes}


def _sizes_from(axes: Mapping[str, int], world: int) -> dict[str, int]:
    sizes = dict(axes)
    if not sizes:
        raise ValueError("axes must name at least one mesh dimension")
    free = [n for n, s in sizes.items() if s == -1]
    if len(free) > 1:
        raise ValueError(f"at most one axis may be -1, got {free}")
    if free:
        fixed = math.prod(s for s in sizes.values() if s != -1)
        if fixed == 0 or world % fixed != 0:
            raise ValueError(
                f"cannot infer -1 axis: world size {world} is not divisible by the product {fixed} of the fixed axes"
            )
        sizes[free[0]] = world // fixed
    bad = {n: s for n, s in sizes.items() if s < 1}
    if bad:
        raise ValueError(f"every axis size must be >= 1, got {bad}")
    return sizes


def _model_axes_from(names: list[str], requested: Sequence[str] | None) -> list[str]:
    if requested is None:
        return list(names)
    req = list(requested)
    if not req:
        raise ValueError("model_parallel_axes must be non-empty when given")
    unknown = [a for a in req if a not in names]
    if unknown:
        raise ValueError(f"model_parallel_axes {unknown} are not in axes {names}")
    if req != names[len(names) - len(req) :]:
        raise ValueError(f"model_parallel_axes must be the trailing axes of {names} in order; got {req}")
    return req


def _resolve_device_type(device_type: str | None) -> str:
    """The device type of the mesh: as given, else what the default group's backend serves (a gloo group
    gets a CPU mesh even where GPUs are present; any other backend gets CUDA when it is available)."""
    if device_type is not None:
        return device_type
    if dist.get_backend() == "gloo":
        return "cpu"
    return "cuda" if torch.cuda.is_available() else "cpu"


def make_process_mesh(
    axes: Mapping[str, int],
    *,
    device_type: str | None = None,
    model_parallel_axes: Sequence[str] | None = None,
    model_key: str = "model",
) -> ProcessMesh:
    """Build a process mesh from ordered ``{axis: size}`` (at most one ``-1``, inferred).

    Needs an initialised default process group on ``nccl``, ``gloo`` or a mix of the two.
    Returns one group per axis plus ``model_key`` spanning ``model_parallel_axes``
    (default: all axes).  The product of the sizes must equal the world size; the error
    is raised identically on every rank.
    """
    if not dist.is_initialized():
        raise RuntimeError(
            "make_process_mesh needs an initialized default process group; call "
            "torch.distributed.init_process_group first"
        )
    check_backend()
    device_type = _resolve_device_type(device_type)
    world = dist.get_world_size()
    sizes = _sizes_from(axes, world)
    names = list(sizes)
    model_axes = _model_axes_from(names, model_parallel_axes)
    if model_key in names:
        raise ValueError(f"model_key {model_key!r} collides with an axis name")
    total = math.prod(sizes.values())
    if total != world:
        raise ValueError(
            f"mesh {dict(sizes)} needs exactly {total} ranks but the process group has {world}; "
            f"launch with {total} ranks or change the axis sizes"
        )
    nd = dist.device_mesh.init_device_mesh(device_type, tuple(sizes.values()), mesh_dim_names=tuple(names))
    mesh = ProcessMesh({n: nd.get_group(n) for n in names}, nd, sizes, model_axes)
    model_n = math.prod(sizes[a] for a in model_axes)
    if len(model_axes) == len(names):
        flat = dist.device_mesh.init_device_mesh(device_type, (model_n,), mesh_dim_names=(model_key,))
    else:
        flat = dist.device_mesh.init_device_mesh(
            device_type, (world // model_n, model_n), mesh_dim_names=("replica", model_key)
        )
    mesh[model_key] = flat.get_group(model_key)
    from .parallel._replicas import register_merged_group

    # every subset of the model axes that tiles the whole replica reduces in one collective
    register_merged_group([mesh[a] for a in model_axes], mesh[model_key])
    return mesh
