#!/usr/bin/env bash
# Held-out cross-entropy / perplexity of a trained checkpoint (one GPU):
#   EXPERIMENT=nestor_200m CHECKPOINT=outputs/nestor_200m/<run>/checkpoints/model_final.pt \
#   VAL_BIN=data/dclm/dclm_val.bin launch/eval.sh
# The trainer's NESTOR eval submission hook (TrainJobConfig.eval_submit_scripts) calls this with the checkpoint
# path as its first argument.
set -euo pipefail
here="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
source "$here/runtime.sh"
EXPERIMENT="${EXPERIMENT:?set EXPERIMENT=<registered experiment>}"
CHECKPOINT="${1:-${CHECKPOINT:?set CHECKPOINT=path/to/model_final.pt}}"
VAL_BIN="${VAL_BIN:?set VAL_BIN=path/to/heldout.bin}"
BLOCK_SIZE="${DCLM_BLOCK_SIZE:-4096}"
MAX_TOKENS="${MAX_TOKENS:-15000000}"
echo "[eval] experiment=${EXPERIMENT} ckpt=${CHECKPOINT} val=${VAL_BIN}"
exec python -m nestor_b200.scripts.eval_heldout --experiment "${EXPERIMENT}" --checkpoint "${CHECKPOINT}" \
  --data "${VAL_BIN}" --block-size "${BLOCK_SIZE}" --max-windows "$(( MAX_TOKENS / BLOCK_SIZE ))" ${OUTPUT:+--output "${OUTPUT}"}
