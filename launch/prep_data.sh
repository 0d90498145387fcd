#!/usr/bin/env bash
# Data preparation (CPU only). One entry point for the four preparation jobs:
#   launch/prep_data.sh pretrain  <dclm shard dir> <out dir>              tokenise DCLM shards into dclm_{train,val}.bin
#   launch/prep_data.sh text      <text/jsonl/parquet files...> --output f.bin          tokenise any text corpus into a .bin
#   launch/prep_data.sh domain    <domain files...> --output data/domain/<name>_train.bin  domain-adaptation corpus
#   launch/prep_data.sh long      <files...> --output data/long/<name>.bin --min-doc-tokens 32768   long-context corpus
#   launch/prep_data.sh replay    seen-subset|replay-mix ...                             derived corpora of the protocols
# Every job writes the flat token file plus its .meta.json sidecar (token count, dtype, eot id, remap).
set -euo pipefail
here="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
job="${1:?pretrain|text|domain|long|replay}"; shift
export TIKTOKEN_CACHE_DIR="${TIKTOKEN_CACHE_DIR:-$(pwd)/data/tiktoken}"
workers="${NUM_WORKERS:-$(nproc)}"
case "$job" in
  pretrain) exec python -m nestor_b200.scripts.preprocess_dclm --dclm-root "${1:?DCLM root}" --out "${2:?output dir}" --workers "$workers" "${@:3}" ;;
  text|domain|long) exec python -m nestor_b200.scripts.preprocess_text_bin --workers "$workers" "$@" ;;
  replay)   exec python -m nestor_b200.scripts.build_corpora "$@" ;;
  *) echo "unknown job: $job" >&2; exit 2 ;;
esac
