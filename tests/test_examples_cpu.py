"""The tutorials under ``examples/``: each runs in-process on 4 gloo ranks (process-group
bring-up replaced by the test's group), the training ones must reduce their loss, the
data-parallel modes must agree with each other, and one script is launched for real with
``torchrun``."""

import importlib
import os
import subprocess
import sys

import pytest
import torch

from dist_utils import run_distributed

EXAMPLES = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples")


def _load(name):
    import torch.distributed as dist

    if EXAMPLES not in sys.path:
        sys.path.insert(0, EXAMPLES)
    common = importlib.import_module("_common")
    common.setup = lambda: (torch.device("cpu"), dist.get_rank(), dist.get_world_size())
    mod = importlib.import_module(name)
    mod.setup = common.setup
    return mod


def _worker_train(rank, world, name, kwargs, steps):
    losses = _load(name).main(steps=steps, **kwargs)
    assert len(losses) == steps and all(v == v for v in losses)
    assert sum(losses[-3:]) < sum(losses[:3]), (name, losses)


@pytest.mark.parametrize("name,kwargs,steps", [
    ("domain_parallel", {}, 12),
    ("vit", {}, 10),
    ("vit", {"ulysses": True}, 6),
    ("swin", {}, 8),
    ("unet3d", {}, 10),
])
def test_training_examples_learn(name, kwargs, steps):
    run_distributed(_worker_train, 4, name, kwargs, steps)


def _worker_selfcheck(rank, world, name, kwargs):
    _load(name).main(**kwargs)


@pytest.mark.parametrize("name,kwargs", [("autoconvert", {}), ("reshard", {"steps": 30}), ("dataloader", {"num_workers": 0}),
                                         ("resume", {"steps": 8})])
def test_self_checking_examples(name, kwargs):
    run_distributed(_worker_selfcheck, 4, name, kwargs)


def _worker_ddp_modes(rank, world):
    import torch.distributed as dist

    vit = _load("vit")
    plain = vit.main(steps=4, data_parallel=True, joint_hook=False)
    joint = vit.main(steps=4, data_parallel=True, joint_hook=True)
    assert max(abs(a - b) for a, b in zip(plain, joint)) < 1e-5, (plain, joint)
    ddp = _load("ddp")
    a = ddp.main(steps=3, joint_hook=True)
    b = ddp.main(steps=3, joint_hook=False)
    assert max(abs(x - y) for x, y in zip(a, b)) < 1e-5, (a, b)


def test_ddp_modes_agree_on_8_ranks():
    run_distributed(_worker_ddp_modes, 8)


def _free_port() -> str:
    import socket

    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        return str(sock.getsockname()[1])


def test_torchrun_launch():
    env = {k: v for k, v in os.environ.items() if not k.startswith("SLURM_")}
    env["CUDA_VISIBLE_DEVICES"] = ""
    env["JIGSAW_LOG_LEVEL"] = "INFO"
    out = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "4", "--master-addr", "127.0.0.1",
         "--master-port", _free_port(), os.path.join(EXAMPLES, "domain_parallel.py"), "--steps", "3"],
        env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-3000:]
    assert "step   0" in out.stderr + out.stdout


def test_cpu_gloo_cnn_workload_matches_undivided_model():
    """The CPU / gloo workload of the benchmarks (four ranks, fp32, two convolutions, Adam): ten steps must
    follow the undivided PyTorch model to rounding."""
    import json

    env = {k: v for k, v in os.environ.items() if not k.startswith("SLURM_")}
    env["CUDA_VISIBLE_DEVICES"] = ""
    script = os.path.join(os.path.dirname(EXAMPLES), "benchmarks", "cpu_cnn.py")
    out = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "4", "--master-addr", "127.0.0.1",
         "--master-port", _free_port(), script, "--steps", "2", "--image", "128"],
        env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-3000:]
    line = [ln for ln in out.stdout.splitlines() if ln.startswith("{")][-1]
    res = json.loads(line)
    assert res["impl"] == "ours" and res["world"] == 4
    assert res["max_loss_diff_vs_undivided"] < 1e-5 and res["max_param_diff_vs_undivided"] < 1e-5
