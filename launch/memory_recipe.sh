#!/usr/bin/env bash
# Memory recipe of a run, by model scale and sequence length; sourced by the launchers after runtime.sh.
#   source launch/memory_recipe.sh <experiment> <sequence length>
# Every flag can be preset in the environment; what is set here are the defaults. A B200 holds 180 GB, so the
# recompute ladder starts later than on the 141 GB parts the reference's recipes were written for
# (scripts/slurm_extend.sh:66-85 of the reference: per-layer checkpointing at 1b, at 64k, and at 500m from 32k):
#   * up to 16k for 100m / 200m and up to 8k for 500m: nothing is recomputed;
#   * 500m from 16k, 200m from 32k, everything at 64k: per-layer regions;
#   * 1b: per-layer regions at every length, split halves from 16k, expert half in 4 row chunks from 32k;
#   * the fused head + cross-entropy is always on (it never materialises [S, vocab] logits).
experiment="${1:?experiment}"; length="${2:-4096}"
scale="${experiment##*_}"
ckpt=0; split=0; chunks=0
case "${scale}:${length}" in
  1b:*) ckpt=1 ;;
  500m:16384|500m:32768|500m:65536) ckpt=1 ;;
  200m:32768|*:65536) ckpt=1 ;;
esac
case "${scale}:${length}" in 1b:16384|1b:32768|1b:65536|500m:65536) split=1 ;; esac
case "${scale}:${length}" in 1b:32768|1b:65536) chunks=4 ;; esac
export NESTOR_ACTIVATION_CHECKPOINT="${NESTOR_ACTIVATION_CHECKPOINT:-$ckpt}"
export NESTOR_ACTIVATION_CHECKPOINT_SPLIT="${NESTOR_ACTIVATION_CHECKPOINT_SPLIT:-$split}"
export NESTOR_EXPERT_HALF_CHUNKS="${NESTOR_EXPERT_HALF_CHUNKS:-$chunks}"
export NESTOR_FUSED_HEAD_CE="${NESTOR_FUSED_HEAD_CE:-1}"
export PYTORCH_CUDA_ALLOC_CONF="${PYTORCH_CUDA_ALLOC_CONF:-expandable_segments:True}"
echo "[memory recipe] ${experiment} @ ${length}: checkpoint=${NESTOR_ACTIVATION_CHECKPOINT} split=${NESTOR_ACTIVATION_CHECKPOINT_SPLIT} expert_chunks=${NESTOR_EXPERT_HALF_CHUNKS} offload=${NESTOR_ACTIVATION_OFFLOAD:-0}"
