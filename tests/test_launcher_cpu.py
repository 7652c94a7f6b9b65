"""``launchers/run.sh`` in ``--dry-run`` mode: the command line and environment it would run under a fake Slurm
allocation, with and without a container, with site presets, and its argument checks.

Reference behaviours covered: scripts/run.sh:36-97 (site presets, validation, rendezvous defaults), :120-167
(bind mounts, forced environment, interpreter choice).
"""

import os
import subprocess
from pathlib import Path

RUN = str(Path(__file__).resolve().parents[1] / "launchers" / "run.sh")


def _run(args, **env):
    base = {"PATH": os.environ["PATH"], "HOME": "/tmp"}
    base.update(env)
    return subprocess.run(["bash", RUN, *args], env=base, capture_output=True, text=True, cwd="/tmp")


def test_local_ranks_become_a_torchrun_command():
    out = _run(["--dry-run", "--local", "4", "python", "bench.py", "--gpus", "4"])
    assert out.returncode == 0, out.stderr
    assert "exec: python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 --master-port 29500 bench.py --gpus 4" in out.stdout
    assert "NCCL_NVLS_ENABLE=1" in out.stdout


def test_slurm_allocation_gives_the_rendezvous_and_a_preset_reaches_the_container():
    out = _run(["--dry-run", "python", "train.py"], JB_SITE="hgx-b200", JB_SIF="/img.sif", JB_BINDS="/a,/b",
               SLURM_JOB_ID="123456", SLURM_JOB_NODELIST="n1", MASTER_ADDR="n1", NCCL_NVLS_ENABLE="0")
    assert out.returncode == 0, out.stderr
    line = [row for row in out.stdout.splitlines() if row.startswith("exec:")][0]
    assert line.startswith("exec: apptainer exec --nv --bind ")
    for piece in ("--bind /a --bind /b", "--env MASTER_ADDR=n1", "--env MASTER_PORT=23456", "--env NCCL_NVLS_ENABLE=0",
                  "--env NCCL_P2P_LEVEL=NVL", "--env JIGSAW_B200_ARENA_SEGMENT_GB=4", "/img.sif python train.py"):
        assert piece in line, (piece, line)


def test_interpreter_override_and_argument_checks(tmp_path):
    out = _run(["--dry-run", "python", "x.py"], JB_PYTHON="/opt/py/bin/python3")
    assert "exec: /opt/py/bin/python3 x.py" in out.stdout
    assert _run([]).returncode == 2
    assert _run(["--local", "zero", "python", "x.py"]).returncode == 2
    assert _run(["--dry-run", "--local", "2", "bash", "x.sh"]).returncode == 2
    missing = _run(["--dry-run", "python", "x.py"], JB_SITE="no-such-cluster")
    assert missing.returncode == 1 and "no site file" in missing.stderr
    bad_venv = _run(["--dry-run", "python", "x.py"], JB_VENV=str(tmp_path))
    assert bad_venv.returncode == 1 and "bin/activate" in bad_venv.stderr
