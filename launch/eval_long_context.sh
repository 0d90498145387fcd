#!/usr/bin/env bash
# Per-position cross-entropy of a (length-extended) checkpoint on long documents (one GPU):
#   EXPERIMENT=nestor_500m CHECKPOINT=<ckpt> VAL_BIN=data/long/pg19_val.bin LENGTH=32768 launch/eval_long_context.sh
# The context length and the matching RoPE base are exported before the registry is imported, because the
# registered cells read them at import time.
set -euo pipefail
here="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
source "$here/runtime.sh"
EXPERIMENT="${EXPERIMENT:?set EXPERIMENT=<registered experiment>}"
CHECKPOINT="${1:-${CHECKPOINT:?set CHECKPOINT=path/to/model.pt}}"
VAL_BIN="${VAL_BIN:?set VAL_BIN=path/to/long_documents.bin}"
LENGTH="${LENGTH:-32768}"
eval "$(python -m nestor_b200.continual.protocols extension --experiment "${EXPERIMENT}" --seq-len "${LENGTH}" \
        --init-checkpoint "${CHECKPOINT}" | grep -E '^export DCLM_ROPE_BASE=' || true)"
echo "[eval-long] experiment=${EXPERIMENT} length=${LENGTH} rope_base=${DCLM_ROPE_BASE:-default} ckpt=${CHECKPOINT}"
exec python -m nestor_b200.scripts.eval_long_context --experiment "${EXPERIMENT}" --checkpoint "${CHECKPOINT}" \
  --data "${VAL_BIN}" --seq-len "${LENGTH}" ${DCLM_ROPE_BASE:+--rope-base "${DCLM_ROPE_BASE}"} \
  --documents "${MAX_SEQUENCES:-64}" ${OUTPUT:+--output "${OUTPUT}"}
