#!/usr/bin/env bash
# Pretrain one registered cell on the GPUs of this node:  launch/pretrain.sh nestor_200m [num_gpus]
# The rung's tokens per step are kept for any GPU count: 4 sequences per GPU, accumulation = rest.
set -euo pipefail
here="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
source "$here/runtime.sh"
experiment="${1:?usage: pretrain.sh <experiment> [num_gpus]}"
gpus="${2:-$(nvidia-smi -L | wc -l)}"
case "$experiment" in
  *_100m) seqs=64 ;; *_200m) seqs=128 ;; *_500m) seqs=256 ;; *_1b) seqs=512 ;; *) seqs="" ;;
esac
per_gpu="${SEQS_PER_GPU:-4}"
if [[ -n "$seqs" && -z "${DCLM_GLOBAL_BATCH:-}" ]]; then
  export DCLM_GLOBAL_BATCH=$((per_gpu * gpus))
  export DCLM_GRAD_ACCUM=$((seqs / DCLM_GLOBAL_BATCH))
fi
source "$here/memory_recipe.sh" "$experiment" "${DCLM_BLOCK_SIZE:-4096}"
export WANDB_MODE="${WANDB_MODE:-disabled}"
exec python -m torch.distributed.run --standalone --local-addr 127.0.0.1 --nproc-per-node "$gpus" \
  -m nestor_b200.cli --experiment "$experiment"
