"""The tutorials as their README tells a user to start them, and the helpers they share.

What is checked without starting a job: the README's table lists exactly the scripts of the folder; every
script defines ``main()`` and calls it only when run as a program (the in-process tests rely on that); the
command-line flags; how many processes and GPUs the node is taken to have, which decides between NCCL and the
CPU.  What starts a job: a script run with bare ``python`` must say how to launch it, and the cheapest script
runs under a real ``torchrun``.

Reference behaviours covered: tests/test_examples_launch.py.
"""

import importlib.util
import os
import re
import subprocess
import sys

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXAMPLES = os.path.join(REPO, "examples")
SCRIPTS = sorted(f[:-3] for f in os.listdir(EXAMPLES) if f.endswith(".py") and not f.startswith("_"))
LAUNCHER_VARIABLES = ("SLURM_", "OMPI_", "PMI_", "PMIX_", "MASTER_", "TORCHELASTIC_", "RANK", "WORLD_SIZE", "LOCAL_RANK",
                      "LOCAL_WORLD_SIZE", "GROUP_RANK")


def _run(args, timeout=600):
    env = {k: v for k, v in os.environ.items() if not k.startswith(LAUNCHER_VARIABLES)}   # nothing of an outer launcher
    env["CUDA_VISIBLE_DEVICES"] = ""
    env["JIGSAW_LOG_LEVEL"] = "INFO"                      # the test session itself runs quieter
    return subprocess.run([sys.executable, *args], cwd=REPO, env=env, capture_output=True, text=True, timeout=timeout)


@pytest.fixture
def common(monkeypatch):
    monkeypatch.syspath_prepend(EXAMPLES)
    spec = importlib.util.spec_from_file_location("examples_common_under_test", os.path.join(EXAMPLES, "_common.py"))
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def test_readme_lists_the_scripts_there_are():
    assert len(SCRIPTS) >= 9
    with open(os.path.join(EXAMPLES, "README.md")) as f:
        listed = re.findall(r"^\| `(\w+)\.py` \|", f.read(), flags=re.MULTILINE)
    assert sorted(listed) == SCRIPTS


@pytest.mark.parametrize("name", SCRIPTS)
def test_script_defines_main_and_guards_it(name):
    with open(os.path.join(EXAMPLES, name + ".py")) as f:
        source = f.read()
    assert "def main(" in source and 'if __name__ == "__main__":' in source
    assert source.lstrip().startswith('"""') and "torchrun --nproc-per-node" in source      # says how to start it


@pytest.mark.parametrize("argv, want", [([], (False, False)), (["--ddp"], (True, False)), (["--joint-hook"], (True, True)),
                                        (["--ddp", "--joint-hook"], (True, True))])
def test_data_parallel_flags(common, argv, want):
    flags = common.ddp_flags(["examples/vit.py", *argv])                                     # the hook needs DDP: it implies it
    assert (flags["data_parallel"], flags["joint_hook"]) == want
    assert common.steps_flag(["x.py", *argv]) == {} and common.steps_flag(["x.py", *argv, "--steps", "7"]) == {"steps": 7}


@pytest.mark.parametrize("env, world, want", [({}, 4, 4), ({"LOCAL_WORLD_SIZE": "4"}, 8, 4), ({"SLURM_NTASKS_PER_NODE": "2"}, 8, 2),
                                              ({"SLURM_NTASKS_PER_NODE": "2(x4)"}, 8, 8)])
def test_processes_on_this_node(common, monkeypatch, env, world, want):
    for var in ("LOCAL_WORLD_SIZE", "SLURM_NTASKS_PER_NODE"):
        monkeypatch.delenv(var, raising=False)
    for var, value in env.items():
        monkeypatch.setenv(var, value)
    assert common._local_processes(world) == want


@pytest.mark.parametrize("visible, env, want", [
    (4, {}, 4), (0, {}, 0), (1, {}, 1),
    (1, {"SLURM_PROCID": "2", "SLURM_STEP_GPUS": "0,1,2,3"}, 4),       # srun bound one GPU to each task
    (1, {"SLURM_PROCID": "0", "SLURM_STEP_GPUS": "0"}, 1),
    (4, {"SLURM_PROCID": "2", "SLURM_STEP_GPUS": "0,1,2,3"}, 4),       # srun, unbound
    (0, {"SLURM_PROCID": "2", "SLURM_STEP_GPUS": "0,1,2,3"}, 0),       # no CUDA at all
    (1, {"SLURM_STEP_GPUS": "0,1,2,3"}, 1),                            # torchrun inside an allocation
])
def test_gpus_on_this_node(common, monkeypatch, visible, env, want):
    for var in ("SLURM_PROCID", "SLURM_STEP_GPUS"):
        monkeypatch.delenv(var, raising=False)
    for var, value in env.items():
        monkeypatch.setenv(var, value)
    monkeypatch.setattr(common.torch.cuda, "device_count", lambda: visible)
    assert common._local_gpus() == want


def test_bare_python_says_how_to_launch():
    out = _run(["examples/domain_parallel.py"], timeout=300)
    assert out.returncode != 0
    assert "needs exactly 4 ranks" in out.stderr and "launch with 4 ranks" in out.stderr, out.stderr[-2000:]


def test_cheapest_script_under_torchrun():
    import socket

    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        port = str(sock.getsockname()[1])
    out = _run(["-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4", "--master-addr", "127.0.0.1", "--master-port", port,
                "examples/dataloader.py", "--steps", "4"])
    assert out.returncode == 0, f"{out.stdout[-2000:]}\n{out.stderr[-4000:]}"
    assert "all checks passed" in out.stdout + out.stderr
