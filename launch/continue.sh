#!/usr/bin/env bash
# Continued training (length extension or domain adaptation) of a pretrained cell:
#   launch/continue.sh extension  nestor_500m --seq-len 32768 --init-checkpoint outputs/nestor_500m
#   launch/continue.sh adaptation nestor_500m --corpus pg19 --replay-pct 25 --init-checkpoint <ckpt>
# Long sequences run one sequence per GPU with activation offload available as a memory lever.
set -euo pipefail
here="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
source "$here/runtime.sh"
kind="${1:?extension|adaptation}"; experiment="${2:?experiment}"; shift 2
gpus="${NUM_GPUS:-$(nvidia-smi -L | wc -l)}"
eval "$(python -m nestor_b200.continual.protocols "$kind" --experiment "$experiment" "$@" | grep '^export')"
export DCLM_GLOBAL_BATCH="${DCLM_GLOBAL_BATCH:-$gpus}"
export DCLM_GRAD_ACCUM="${DCLM_GRAD_ACCUM:-$((CONTINUAL_SEQS_PER_STEP / DCLM_GLOBAL_BATCH))}"
export NESTOR_ACTIVATION_OFFLOAD="${NESTOR_ACTIVATION_OFFLOAD:-0}"
source "$here/memory_recipe.sh" "$experiment" "${DCLM_BLOCK_SIZE:-4096}"
export WANDB_MODE="${WANDB_MODE:-disabled}"
exec python -m torch.distributed.run --standalone --local-addr 127.0.0.1 --nproc-per-node "$gpus" \
  -m nestor_b200.cli --experiment "$experiment"
