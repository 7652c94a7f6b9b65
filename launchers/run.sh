#!/usr/bin/env bash
# Launcher for B200 nodes: run one command per GPU, bare-metal or inside a container.
#
#   launchers/run.sh python examples/vit.py                      # under srun: one task per GPU
#   JB_SITE=mycluster srun --ntasks-per-node=8 launchers/run.sh python bench.py --gpus 8
#   launchers/run.sh --local 8 python bench.py --gpus 8          # no scheduler: torchrun on this node
#
# Site settings come from launchers/sites/<JB_SITE>.env or $JB_SITE_FILE (both optional):
#   JB_SIF        container image (.sif); unset = run on the host
#   JB_RUNTIME    container runtime (default: apptainer)
#   JB_BINDS      comma-separated bind mounts
#   JB_VENV       virtual environment to activate
#   JB_MODULES    modules to load first
#
# What jigsaw_b200.launch needs: SLURM_PROCID / SLURM_NTASKS / SLURM_LOCALID (srun) or RANK /
# WORLD_SIZE / LOCAL_RANK (torchrun), and MASTER_ADDR / MASTER_PORT.  Under SLURM the two MASTER_
# variables are derived from the allocation when unset.
set -euo pipefail
here="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
root="$(dirname "$here")"

local_ranks=0
if [[ "${1:-}" == "--local" ]]; then
    local_ranks="$2"; shift 2
fi
if [[ $# -eq 0 ]]; then
    echo "usage: run.sh [--local N] <command ...>" >&2; exit 2
fi

site_file="${JB_SITE_FILE:-}"
if [[ -z "$site_file" && -n "${JB_SITE:-}" ]]; then site_file="$here/sites/${JB_SITE}.env"; fi
if [[ -n "$site_file" ]]; then
    if [[ ! -r "$site_file" ]]; then echo "run.sh: no site file $site_file" >&2; exit 1; fi
    # shellcheck disable=SC1090
    source "$site_file"
fi
if [[ -n "${JB_MODULES:-}" ]] && command -v module >/dev/null 2>&1; then
    for m in $JB_MODULES; do module load "$m"; done
fi

# rendezvous: first host of the allocation, a port derived from the job id
if [[ -n "${SLURM_JOB_ID:-}" ]]; then
    if [[ -z "${MASTER_ADDR:-}" ]]; then
        MASTER_ADDR="$(scontrol show hostnames "${SLURM_JOB_NODELIST}" | head -n1)"; export MASTER_ADDR
    fi
    export MASTER_PORT="${MASTER_PORT:-$((20000 + SLURM_JOB_ID % 20000))}"
fi

# NVLink / NVSwitch domain defaults (all overridable from the environment)
export NCCL_NVLS_ENABLE="${NCCL_NVLS_ENABLE:-1}"          # in-switch reductions
export TORCH_NCCL_ASYNC_ERROR_HANDLING="${TORCH_NCCL_ASYNC_ERROR_HANDLING:-1}"
export CUDA_DEVICE_MAX_CONNECTIONS="${CUDA_DEVICE_MAX_CONNECTIONS:-8}"
export PYTHONPATH="$root${PYTHONPATH:+:$PYTHONPATH}"

cmd=("$@")
if [[ "$local_ranks" -gt 0 ]]; then
    cmd=(python -m torch.distributed.run --nnodes=1 --nproc-per-node "$local_ranks" --master-addr 127.0.0.1
         --master-port "${MASTER_PORT:-29500}" "${@:2}")
    if [[ "$1" != "python" ]]; then echo "run.sh: --local expects 'python <script> ...'" >&2; exit 2; fi
fi
if [[ -n "${JB_VENV:-}" ]]; then
    # shellcheck disable=SC1091
    source "$JB_VENV/bin/activate"
fi
if [[ -n "${JB_SIF:-}" ]]; then
    binds=()
    if [[ -n "${JB_BINDS:-}" ]]; then binds=(--bind "$JB_BINDS"); fi
    exec "${JB_RUNTIME:-apptainer}" exec --nv "${binds[@]}" --bind "$root" "$JB_SIF" "${cmd[@]}"
fi
exec "${cmd[@]}"
