"""What becomes of the reference's environment flags here.

The reference selects its execution paths with ``NESTOR_*`` variables (its speed stack exports about thirty of
them). This framework has one kernel path per op, so most of those switches have nothing to select; a launcher
written for the reference can be reused unchanged, and ``report_reference_flags`` tells the user at start-up which of
the variables it exports are read, which have no effect, and which ask for something that works differently here.
The catalogue follows the reference's flag list (``scripts/lib/speed_stack.sh:14-35`` and the modules named there).
"""

from __future__ import annotations

import logging
import os
from typing import Mapping

# Fast-path selectors of the reference's PyTorch / Triton implementations: the kernel path is always on here.
NO_EFFECT: dict[str, str] = {
    **{k: "attention always runs the packed variable-length kernels" for k in (
        "NESTOR_ATTN_PACKED_VARLEN", "NESTOR_TRITON_PACKED_ATTN", "NESTOR_PACKED_POINTWISE_COMPILE",
        "NESTOR_DENSE_TAIL_ATTN", "NESTOR_GATHERED_CAUSAL_FLASH", "NESTOR_GATHERED_VARLEN", "NESTOR_GROUPED_ATTN_BMM",
        "NESTOR_GROUPED_PROJ_BMM", "NESTOR_GATHERED_CAP_BUCKET", "NESTOR_STATIC_CAPACITY_FRAC", "NESTOR_ATTN_CAUSAL_SDPA",
        "NESTOR_DENSE_FULL_ATTN", "NESTOR_FORCE_NO_TOKEN_DISPATCH", "NESTOR_CAUSAL_FULL_QCHUNK",
        "NESTOR_NO_DENSE_FASTPATH", "NESTOR_DENSE_TAIL_QUERY_CHUNKS", "NESTOR_STACKED_ATTN_WEIGHTS",
        "NESTOR_BATCHED_ATTN_COMPILE")},
    **{k: "experts always run the grouped tensor-core products with in-kernel dispatch plans" for k in (
        "NESTOR_MOE_GROUPED_MM", "NESTOR_POOL_GROUPED_MM", "NESTOR_GROUPED_MM_FUSED_GATE", "NESTOR_TRITON_INDEX_BUILD",
        "NESTOR_TRITON_EXPERT_DISPATCH", "NESTOR_TRITON_EXPERT_CATCAST", "NESTOR_BATCHED_ROUTERS")},
    **{k: "column streams are always kept in slot layout with one fused update per layer" for k in (
        "NESTOR_COLUMN_SLOT_UPDATES", "NESTOR_COLUMN_FUSE_SCATTER")},
    **{k: "nothing is traced or compiled: kernels are built ahead of time and the micro-batch is a CUDA graph" for k in (
        "NESTOR_COMPILE", "NESTOR_COMPILE_MODE", "NESTOR_RECOMPILE_LIMIT", "NESTOR_NO_PERSISTENT_REDUCTIONS",
        "NESTOR_PREWARM_CAUSAL_SEQ", "NESTOR_COMPILED_EVAL", "NESTOR_DEPTH_READ_EAGER", "NESTOR_DEPTH_READ_COMPILE_MAX",
        "NESTOR_DEPTH_READ_AUTOCAST")},
    **{k: "gradients live in one arena that is reduced once per optimizer step" for k in (
        "NESTOR_DDP_NO_SYNC", "NESTOR_DDP_STATIC_GRAPH", "NESTOR_DDP_FIND_UNUSED")},
    "NESTOR_BF16_MASTER": "bf16 compute with fp32 masters is the only bf16 mode",
}

# Values that ask for a mode with a different equivalent here: (variable, value that triggers the note, note).
DIFFERENT: tuple[tuple[str, str, str], ...] = (
    ("NESTOR_DDP", "0", "FSDP2 parameter sharding is not built: the run is data parallel with ZeRO-1 optimizer state "
                        "(NESTOR_MUON_SHARD / NESTOR_ZERO1) and, optionally, rank-sharded expert-bank reads (NESTOR_FSDP_BANKS)"),
    ("NESTOR_DISABLE_FSDP", "0", "FSDP2 parameter sharding is not built (see NESTOR_DDP)"),
    ("NESTOR_FSDP_RESHARD", "1", "there is no per-block parameter gather to reshard"),
    ("NESTOR_STACKED_EXPERT_BANKS", "0", "expert banks are always stacked; per-expert checkpoints are converted on load"),
    ("NESTOR_DENSE_NO_ROUTER", "0", "single-choice routers are always frozen and skipped"),
)


def classify(env: Mapping[str, str] | None = None) -> dict[str, dict[str, str]]:
    """``{"no_effect": {name: why}, "different": {name: note}}`` for the variables set in ``env``."""

    env = os.environ if env is None else env
    out: dict[str, dict[str, str]] = {"no_effect": {}, "different": {}}
    for name, why in NO_EFFECT.items():
        if env.get(name, "") != "":
            out["no_effect"][name] = why
    for name, value, note in DIFFERENT:
        if env.get(name) == value:
            out["different"][f"{name}={value}"] = note
    return out


def report_reference_flags(logger: logging.Logger, env: Mapping[str, str] | None = None) -> dict[str, dict[str, str]]:
    """Log, once at start-up, which exported reference flags have no effect here and which mean something else."""

    found = classify(env)
    if found["no_effect"]:
        reasons: dict[str, list[str]] = {}
        for name, why in found["no_effect"].items():
            reasons.setdefault(why, []).append(name)
        for why, names in reasons.items():
            logger.info("[flags] no effect here (%s): %s", why, " ".join(sorted(names)))
    for what, note in found["different"].items():
        logger.warning("[flags] %s: %s", what, note)
    return found
