"""Shared by the tutorials: bring-up of the process group, input sharding, command-line flags."""

from __future__ import annotations

import atexit
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))   # run from a checkout

from jigsaw_b200 import launch, log  # noqa: E402


def _local_processes(world: int) -> int:
    for var in ("LOCAL_WORLD_SIZE", "SLURM_NTASKS_PER_NODE"):
        if os.environ.get(var, "").isdigit():
            return int(os.environ[var])
    return world


def _local_gpus() -> int:
    n = torch.cuda.device_count()
    bound = os.environ.get("SLURM_STEP_GPUS", "")
    if n == 1 and bound and "SLURM_PROCID" in os.environ:       # srun bound one GPU to each task
        n = len(bound.split(","))
    return n


def _shutdown() -> None:
    if dist.is_initialized():
        dist.destroy_process_group()


def setup() -> tuple[torch.device, int, int]:
    """``(device, rank, world_size)``: NCCL with one GPU per process when the node has enough
    GPUs, otherwise gloo on the CPU (same command line, e.g. on a laptop)."""
    atexit.register(_shutdown)
    env = launch.resolve_launch_env()
    gpus = _local_gpus()
    if gpus and gpus >= _local_processes(env.world_size):
        device, _, rank, world = launch.init_cuda()
        return device, rank, world
    log.configure_logging()
    if gpus:
        log.info("%d GPU(s) for %d processes: running on the CPU", gpus, env.world_size)
    os.environ.setdefault("MASTER_ADDR", env.master_addr)
    os.environ.setdefault("MASTER_PORT", env.master_port)
    dist.init_process_group("gloo", rank=env.rank, world_size=env.world_size, init_method="env://")
    return torch.device("cpu"), env.rank, env.world_size


def shard(x: torch.Tensor, dim: int, group: dist.ProcessGroup) -> torch.Tensor:
    """This rank's block of ``x`` along ``dim`` when it is cut over ``group``."""
    n = x.shape[dim] // group.size()
    return x.narrow(dim, group.rank() * n, n).contiguous()


def ddp_flags(argv: list[str]) -> dict[str, bool]:
    """``--ddp`` adds a data-parallel axis; ``--joint-hook`` does too and reduces through the joint hook."""
    joint = "--joint-hook" in argv
    return {"data_parallel": joint or "--ddp" in argv, "joint_hook": joint}


def steps_flag(argv: list[str]) -> dict[str, int]:
    return {"steps": int(argv[argv.index("--steps") + 1])} if "--steps" in argv else {}


def data_seed(step: int, mesh) -> int:
    """Batch seed: equal within a model copy (its ranks cut up the same samples), distinct
    across data-parallel copies."""
    dp = mesh.get("dp")
    return step if dp is None else step * dp.size() + dp.rank()


def denoising_batch(step: int, mesh, shape: tuple[int, ...]) -> tuple[torch.Tensor, torch.Tensor]:
    """A smooth random field and a noisy version of it (global tensors, same on the ranks of a copy)."""
    g = torch.Generator().manual_seed(data_seed(step, mesh))
    clean = torch.nn.functional.avg_pool2d(torch.randn(*shape, generator=g), 5, 1, 2)
    return clean + 0.3 * torch.randn(clean.shape, generator=g), clean


def train(model, loss_fn, batch_fn, steps: int, lr: float = 1e-3) -> list[float]:
    """Plain AdamW loop; ``batch_fn(step)`` returns this rank's ``(input, target)``."""
    opt = torch.optim.AdamW(model.parameters(), lr=lr)
    losses = []
    for step in range(steps):
        x, y = batch_fn(step)
        loss = loss_fn(model(x), y)
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(loss.item())
        if step % 20 == 0:
            log.info("step %3d  loss %.4f", step, losses[-1])
    return losses
