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
#   JB_PYTHON     interpreter that replaces a bare "python" / "python3" when no venv is set
#   JB_ENV_FILE   extra --env-file handed to the container runtime
#   JB_PASS_ENV   space-separated names of further variables to force into the container
#
# Options (before the command):
#   --local N     no scheduler: start N ranks on this node with torchrun
#   --dry-run     print the resolved environment and the command line instead of running it
#
# What jigsaw_b200.launch needs: SLURM_PROCID / SLURM_NTASKS / SLURM_LOCALID (srun) or RANK /
# WORLD_SIZE / LOCAL_RANK (torchrun), and MASTER_ADDR / MASTER_PORT.  Under SLURM the two MASTER_
# variables are derived from the allocation when unset.
set -euo pipefail
here="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
root="$(dirname "$here")"

local_ranks=0
dry_run=0
while [[ $# -gt 0 ]]; do
    case "$1" in
        --local)
            if [[ ! "${2:-}" =~ ^[1-9][0-9]*$ ]]; then echo "run.sh: --local needs a positive rank count" >&2; exit 2; fi
            local_ranks="$2"; shift 2 ;;
        --dry-run) dry_run=1; shift ;;
        --) shift; break ;;
        *) break ;;
    esac
done
if [[ $# -eq 0 ]]; then
    echo "usage: run.sh [--local N] [--dry-run] <command ...>" >&2; exit 2
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
    if [[ ! -r "$JB_VENV/bin/activate" ]]; then echo "run.sh: JB_VENV=$JB_VENV has no bin/activate" >&2; exit 1; fi
    if [[ "$dry_run" -eq 0 ]]; then
        # shellcheck disable=SC1091
        source "$JB_VENV/bin/activate"
    fi
elif [[ -n "${JB_PYTHON:-}" && ( "${cmd[0]}" == "python" || "${cmd[0]}" == "python3" ) ]]; then
    cmd[0]="$JB_PYTHON"
fi
if [[ -n "${JB_SIF:-}" ]]; then
    if [[ "$dry_run" -eq 0 && ! -r "$JB_SIF" ]]; then echo "run.sh: container image $JB_SIF is not readable" >&2; exit 1; fi
    runtime="${JB_RUNTIME:-apptainer}"
    if [[ "$dry_run" -eq 0 ]] && ! command -v "$runtime" >/dev/null 2>&1; then
        echo "run.sh: container runtime '$runtime' not found (set JB_RUNTIME, or unset JB_SIF to run on the host)" >&2; exit 1
    fi
    binds=(--bind "$root")
    IFS=',' read -r -a extra_binds <<< "${JB_BINDS:-}"
    for b in "${extra_binds[@]}"; do [[ -n "$b" ]] && binds+=(--bind "$b"); done
    env_file=()
    [[ -n "${JB_ENV_FILE:-}" ]] && env_file=(--env-file "$JB_ENV_FILE")
    # images may bake their own values into %environment, which beat plain passthrough: force ours with --env
    forced=()
    for v in MASTER_ADDR MASTER_PORT NCCL_NVLS_ENABLE TORCH_NCCL_ASYNC_ERROR_HANDLING CUDA_DEVICE_MAX_CONNECTIONS \
             NCCL_DEBUG JIGSAW_STRICT_FUSED JIGSAW_LOG_LEVEL JIGSAW_LOG_DIR JIGSAW_LOG_FORMAT ${JB_PASS_ENV:-}; do
        [[ -n "${!v:-}" ]] && forced+=(--env "$v=${!v}")
    done
    cmd=("$runtime" exec --nv "${binds[@]}" "${env_file[@]}" "${forced[@]}" --env "PYTHONPATH=$PYTHONPATH" "$JB_SIF" "${cmd[@]}")
fi
if [[ "$dry_run" -eq 1 ]]; then
    for v in MASTER_ADDR MASTER_PORT NCCL_NVLS_ENABLE CUDA_DEVICE_MAX_CONNECTIONS PYTHONPATH; do echo "$v=${!v:-}"; done
    printf 'exec:'; printf ' %q' "${cmd[@]}"; printf '\n'
    exit 0
fi
exec "${cmd[@]}"
