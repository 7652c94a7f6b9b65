"""Process launch and runtime set-up: launcher detection, device selection, seeds, TF32.

Launcher precedence: SLURM (``SLURM_PROCID`` / ``SLURM_NTASKS`` / ``SLURM_LOCALID``),
then torchrun (``RANK`` / ``WORLD_SIZE`` / ``LOCAL_RANK``), then a single process.

Reference parity: jigsaw/launch.py:21-31 (seeds), :34-114 (launch env), :117-164
(init_cuda), :167-177 (TF32 switch).
"""

from __future__ import annotations

import os
import subprocess
from dataclasses import dataclass

import torch
import torch.distributed as dist

from . import log

__all__ = ["LaunchEnv", "init_cuda", "init_cpu", "resolve_launch_env", "set_all_seeds", "setup_precision"]


def set_all_seeds(seed: int = 0) -> None:
    """Seed the CPU and every CUDA generator of PyTorch."""
    os.environ["PL_GLOBAL_SEED"] = str(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


@dataclass(frozen=True)
class LaunchEnv:
    """Where this process sits in the job and how the ranks find each other."""

    rank: int
    world_size: int
    local_rank: int
    master_addr: str
    master_port: str
    source: str  # which launcher's variables were found: "slurm", "torchrun", "mpirun" or "single"


# launcher name -> the variables that carry (rank, world size, local rank); the first launcher whose rank
# variable is set wins, so an srun step started from inside a torchrun shell is read as Slurm
_LAUNCHERS = (
    ("slurm", ("SLURM_PROCID", "SLURM_NTASKS", "SLURM_LOCALID")),
    ("torchrun", ("RANK", "WORLD_SIZE", "LOCAL_RANK")),
    ("mpirun", ("OMPI_COMM_WORLD_RANK", "OMPI_COMM_WORLD_SIZE", "OMPI_COMM_WORLD_LOCAL_RANK")),      # Open MPI
)


def _first_slurm_host(nodelist: str) -> str:
    hosts = subprocess.check_output(["scontrol", "show", "hostnames", nodelist]).decode().split()
    return hosts[0]


def resolve_launch_env(strict: bool = False) -> LaunchEnv:
    """Work out rank, world size and local rank from the launcher's environment variables, and the rendezvous
    address and port, which are also exported (``MASTER_ADDR`` / ``MASTER_PORT``) so that ``init_method="env://"``
    finds them.

    The address is taken as given, else it is the first host of the Slurm allocation (``scontrol show hostnames``),
    else ``localhost``; the port defaults to 29500.  A launcher that sets only its rank variable gets a world of one
    and local rank 0; a rank variable that is set but empty is an error of the launcher and raises ``ValueError``.
    Without any launcher this is a single process, or a ``RuntimeError`` when ``strict`` is set.
    """
    env = os.environ
    for source, (rank_var, world_var, local_var) in _LAUNCHERS:
        if rank_var in env:
            rank = int(env[rank_var])
            world = int(env.get(world_var) or 1)
            local = int(env.get(local_var) or 0)
            break
    else:
        if strict:
            raise RuntimeError(
                "No distributed launcher detected: expected SLURM_PROCID (srun), RANK (torchrun) or "
                "OMPI_COMM_WORLD_RANK (mpirun) in the environment. Launch with one of them, or pass strict=False for a "
                "single-process run."
            )
        source, rank, world, local = "single", 0, 1, 0
    addr = env.get("MASTER_ADDR") or (_first_slurm_host(env["SLURM_JOB_NODELIST"]) if env.get("SLURM_JOB_NODELIST") else "localhost")
    port = env.get("MASTER_PORT") or "29500"
    env["MASTER_ADDR"], env["MASTER_PORT"] = addr, port
    return LaunchEnv(rank, world, local, addr, port, source)


def init_cuda() -> tuple[torch.device, int, int, int]:
    """Pick the local GPU, start the NCCL process group, return ``(device, local_rank, rank, world_size)``."""
    e = resolve_launch_env()
    log.configure_logging()
    log.info_all("launch: rank %d/%d, local_rank %d, via %s", e.rank, e.world_size, e.local_rank, e.source)
    index = e.local_rank if torch.cuda.device_count() != 1 else 0
    device = torch.device("cuda", index)
    torch.cuda.set_device(index)
    dist.init_process_group(
        backend="nccl", rank=e.rank, world_size=e.world_size, init_method="env://", device_id=device
    )
    log.info(
        "process group up: torch rank %d, world size %d, backend %s",
        dist.get_rank(),
        dist.get_world_size(),
        dist.get_backend(),
    )
    return device, e.local_rank, e.rank, e.world_size


def init_cpu() -> tuple[torch.device, int, int, int]:
    """Gloo counterpart of :func:`init_cuda` for CPU runs (tests, laptops)."""
    e = resolve_launch_env()
    log.configure_logging()
    dist.init_process_group(backend="gloo", rank=e.rank, world_size=e.world_size, init_method="env://")
    return torch.device("cpu"), e.local_rank, e.rank, e.world_size


def setup_precision(tf32: bool) -> None:
    """Allow or forbid TF32 in cuBLAS matmuls and cuDNN convolutions."""
    torch.backends.cuda.matmul.allow_tf32 = bool(tf32)
    torch.backends.cudnn.allow_tf32 = bool(tf32)
