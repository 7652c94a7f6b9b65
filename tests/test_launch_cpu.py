"""Launch contract: rendezvous address and port (explicit, derived from the Slurm node list, defaults, written back
for ``env://``), missing optional variables, the frozen result object, and which CUDA device a process takes
(CUDA and the process group faked).

Reference behaviours covered: tests/test_launch_env.py:119-148 (defaults), :150-218 (address, port, write-back),
:220-230 (result object), :232-272 (device choice).
"""

import dataclasses
import os
import types

import pytest

from jigsaw_b200 import launch

VARS = ("SLURM_PROCID", "SLURM_NTASKS", "SLURM_LOCALID", "SLURM_JOB_NODELIST", "RANK", "WORLD_SIZE", "LOCAL_RANK",
        "OMPI_COMM_WORLD_RANK", "OMPI_COMM_WORLD_SIZE", "OMPI_COMM_WORLD_LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT")


@pytest.fixture(autouse=True)
def _clean(monkeypatch):
    for name in VARS:
        monkeypatch.delenv(name, raising=False)
    yield
    for name in ("MASTER_ADDR", "MASTER_PORT"):            # resolve_launch_env writes them back
        os.environ.pop(name, None)


def _fake_scontrol(monkeypatch, output):
    calls = []

    def check_output(cmd, *args, **kwargs):
        calls.append(cmd)
        return output

    monkeypatch.setattr(launch.subprocess, "check_output", check_output)
    return calls


def test_missing_optional_variables_fall_back(monkeypatch):
    monkeypatch.setenv("SLURM_PROCID", "0")
    env = launch.resolve_launch_env()
    assert (env.source, env.world_size, env.local_rank) == ("slurm", 1, 0)
    monkeypatch.delenv("SLURM_PROCID")
    monkeypatch.setenv("RANK", "0")
    env = launch.resolve_launch_env()
    assert (env.source, env.world_size, env.local_rank) == ("torchrun", 1, 0)
    monkeypatch.setenv("SLURM_PROCID", "")                   # set but empty: the Slurm branch is taken and refuses it
    with pytest.raises(ValueError):
        launch.resolve_launch_env()


def test_master_address_explicit_derived_and_default(monkeypatch):
    monkeypatch.setenv("MASTER_ADDR", "10.0.0.5")
    monkeypatch.setenv("SLURM_JOB_NODELIST", "node[01-04]")
    calls = _fake_scontrol(monkeypatch, b"node01\n")
    assert launch.resolve_launch_env().master_addr == "10.0.0.5" and calls == []
    monkeypatch.delenv("MASTER_ADDR")
    monkeypatch.setenv("SLURM_PROCID", "0")
    monkeypatch.setenv("SLURM_NTASKS", "4")
    calls = _fake_scontrol(monkeypatch, b"node01\nnode02\nnode03\nnode04\n")
    env = launch.resolve_launch_env()
    assert env.master_addr == "node01" and calls == [["scontrol", "show", "hostnames", "node[01-04]"]]
    assert os.environ["MASTER_ADDR"] == "node01"
    monkeypatch.delenv("MASTER_ADDR")
    monkeypatch.delenv("SLURM_JOB_NODELIST")
    assert launch.resolve_launch_env().master_addr == "localhost"


def test_master_port_default_override_and_write_back(monkeypatch):
    env = launch.resolve_launch_env()
    assert env.master_port == "29500" == os.environ["MASTER_PORT"] and os.environ["MASTER_ADDR"] == "localhost"
    monkeypatch.setenv("MASTER_PORT", "12321")
    monkeypatch.setenv("MASTER_ADDR", "10.1.2.3")
    env = launch.resolve_launch_env()
    assert (env.master_addr, env.master_port) == ("10.1.2.3", "12321") == (os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"])


def test_the_result_is_an_immutable_value():
    env = launch.resolve_launch_env()
    assert isinstance(env, launch.LaunchEnv)
    with pytest.raises(dataclasses.FrozenInstanceError):
        env.rank = 99


@pytest.mark.parametrize("visible, local_rank, expected", [(4, 0, 0), (4, 3, 3), (1, 0, 0), (1, 3, 0)])
def test_device_choice(monkeypatch, visible, local_rank, expected):
    """Every process sees the node's GPUs: one each, by local rank; the launcher bound one GPU per task: always 0."""
    monkeypatch.setenv("SLURM_PROCID", str(4 + local_rank))
    monkeypatch.setenv("SLURM_NTASKS", "8")
    monkeypatch.setenv("SLURM_LOCALID", str(local_rank))
    monkeypatch.setenv("MASTER_ADDR", "node0")
    selected, started = [], []
    monkeypatch.setattr(launch.torch.cuda, "device_count", lambda: visible)
    monkeypatch.setattr(launch.torch.cuda, "set_device", selected.append)
    monkeypatch.setattr(launch.dist, "init_process_group", lambda **kw: started.append(kw))
    monkeypatch.setattr(launch.dist, "get_rank", lambda: 4 + local_rank)
    monkeypatch.setattr(launch.dist, "get_world_size", lambda: 8)
    monkeypatch.setattr(launch.dist, "get_backend", lambda: "nccl")
    noop = lambda *a, **k: None                                  # noqa: E731
    monkeypatch.setattr(launch, "log", types.SimpleNamespace(configure_logging=noop, info_all=noop, info=noop, error_all=noop))
    device, got_local, rank, world = launch.init_cuda()
    assert (device.type, device.index) == ("cuda", expected) and selected == [expected]
    assert (got_local, rank, world) == (local_rank, 4 + local_rank, 8)   # the local rank is reported as launched
    assert started[0]["backend"] == "nccl" and started[0]["rank"] == 4 + local_rank and started[0]["world_size"] == 8


def test_open_mpi_variables_come_last(monkeypatch):
    """``mpirun`` (Open MPI) is read when neither Slurm nor torchrun variables are there; either of those wins."""
    for name, value in (("OMPI_COMM_WORLD_RANK", "5"), ("OMPI_COMM_WORLD_SIZE", "8"), ("OMPI_COMM_WORLD_LOCAL_RANK", "1")):
        monkeypatch.setenv(name, value)
    env = launch.resolve_launch_env(strict=True)
    assert (env.source, env.rank, env.world_size, env.local_rank) == ("mpirun", 5, 8, 1)
    assert (env.master_addr, env.master_port) == ("localhost", "29500")
    monkeypatch.setenv("RANK", "2")
    monkeypatch.setenv("WORLD_SIZE", "4")
    assert launch.resolve_launch_env().source == "torchrun"
    monkeypatch.setenv("SLURM_PROCID", "3")
    assert launch.resolve_launch_env().source == "slurm"
