"""``make_process_mesh``: validation (every refusal before any group is made, the same on every rank), inference of
one ``-1`` axis, the model group over the trailing model-parallel axes, the n-d device mesh behind the groups.

Reference behaviours covered: tests/test_mesh.py:7-93 (validation, device type), :95-125 (four-rank layouts).
"""

import pytest
import torch

from dist_utils import run_distributed


def _worker_mesh(rank, world):
    import jigsaw_b200 as jb
    import torch.distributed as dist

    make = jb.make_process_mesh
    mesh = make({"col": world})
    assert set(mesh) == {"col", "model"} and mesh["col"].size() == world == mesh["model"].size()
    assert make({"dp": -1, "row": 1, "col": 1})["dp"].size() == world
    for axes, kw, pattern in (
        ({"row": world + 1}, {}, r"needs exactly \d+ ranks"),
        ({"a": -1, "b": -1}, {}, "at most one axis may be -1"),
        ({"row": 1, "col": 1}, {"model_parallel_axes": ("row",)}, "trailing axes"),
        ({"model": 1}, {}, "collides with an axis"),
        ({}, {}, "at least one mesh dimension"),
        ({"a": -1, "b": 0}, {}, "cannot infer -1 axis"),
        ({"a": -1, "b": world + 1}, {}, "cannot infer -1 axis"),
        ({"a": 0}, {}, "every axis size must be >= 1"),
        ({"a": -2}, {}, "every axis size must be >= 1"),
        ({"a": -1}, {"model_parallel_axes": ()}, "must be non-empty"),
        ({"a": -1}, {"model_parallel_axes": ("nope",)}, "are not in axes"),
    ):
        with pytest.raises(ValueError, match=pattern):
            make(axes, **kw)
    # four ranks: fully model-parallel, a replica axis outside the model group, spatial axes inside it
    mesh = make({"row": 2, "col": 2})
    assert (mesh["row"].size(), mesh["col"].size(), mesh["model"].size()) == (2, 2, 4)
    assert mesh["model"].rank() == mesh["row"].rank() * 2 + mesh["col"].rank()           # row-major rank inside the model group
    mesh = make({"dp": 2, "row": 1, "col": 2}, model_parallel_axes=("row", "col"))
    assert mesh["dp"].size() == 2 and mesh["model"].size() == 2 and isinstance(mesh, dict)
    assert mesh.device_mesh.mesh_dim_names == ("dp", "row", "col")
    for name in ("dp", "row", "col"):
        sliced = mesh.device_mesh[name].get_group()
        assert dist.get_process_group_ranks(sliced) == dist.get_process_group_ranks(mesh[name])
    mesh = make({"sh": 2, "sw": 2, "col": 1})
    assert (mesh["sh"].size(), mesh["sw"].size(), mesh["col"].size(), mesh["model"].size()) == (2, 2, 1, 4)
    mesh = make({"dp": 2, "row": 2, "col": 1}, model_parallel_axes=("row", "col"), model_key="mp")
    assert "mp" in mesh and "model" not in mesh and mesh["mp"].size() == 2


def test_mesh_validation_and_layouts():
    run_distributed(_worker_mesh, 4, timeout=300)


def test_mesh_needs_a_process_group_and_a_supported_backend(monkeypatch):
    import torch.distributed as dist

    import jigsaw_b200 as jb
    from jigsaw_b200 import mesh

    monkeypatch.setattr(dist, "is_initialized", lambda: False)
    with pytest.raises(RuntimeError, match="initialized default process group"):
        jb.make_process_mesh({"a": 1})
    monkeypatch.setattr(dist, "is_initialized", lambda: True)
    monkeypatch.setattr(dist, "get_backend", lambda group=None: "mpi")
    with pytest.raises(RuntimeError, match="unsupported process-group backend"):
        jb.make_process_mesh({"a": -1})
    # the device type follows the default group's backend, not the hardware that happens to be present
    monkeypatch.setattr(dist, "get_backend", lambda group=None: "nccl")
    monkeypatch.setattr(torch.cuda, "is_available", lambda: False)
    assert mesh._resolve_device_type(None) == "cpu"
    monkeypatch.setattr(torch.cuda, "is_available", lambda: True)
    assert mesh._resolve_device_type(None) == "cuda" and mesh._resolve_device_type("cpu") == "cpu"
    monkeypatch.setattr(dist, "get_backend", lambda group=None: "gloo")
    assert mesh._resolve_device_type(None) == "cpu" and mesh._resolve_device_type("cuda") == "cuda"
