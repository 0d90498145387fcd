"""Analytic forward FLOPs of the registered models at any context length.

Accounting rules (same as the reference's ``nestor/continual/flops.py:1-25``): per layer of
a block with ``G`` columns, ``k`` active, column width ``w``, sequence length ``S``:
projections ``8 S d w k``; causal core ``G * 2 (S k / G)^2 w`` (4 instead of 2 when not
causal), assuming balanced routing; SwiGLU MLP ``6 S d * active_width`` where the active
width is ``top_k * width`` for a bank and ``k_p h_pub + k k_q h_priv`` for the hybrid pool.
Routers, depth reads, norms and the LM head are excluded from the *body*; the head is
available separately for MFU accounting.
"""

from __future__ import annotations

import dataclasses as dc

from nestor_b200.configs.model import NestorConfig
from nestor_b200.experiments.pretrain import ARMS, SCALES

FAMILIES = ("dense", "moe", "nestor")


@dc.dataclass(frozen=True)
class BodyFlops:
    projections: float
    core: float
    mlp: float

    @property
    def total(self) -> float:
        return self.projections + self.core + self.mlp


def split_experiment_name(experiment: str) -> tuple[str, str]:
    family, _, scale = experiment.rpartition("_")
    if family not in FAMILIES or scale not in SCALES:
        raise ValueError(f"{experiment!r} is not a registered cell (<family>_<scale>).")
    return family, scale


def experiment_backbone(experiment: str) -> NestorConfig:
    family, scale = split_experiment_name(experiment)
    return ARMS[family](SCALES[scale])


def backbone_body_flops(backbone: NestorConfig, *, seq_len: int, causal: bool = True) -> BodyFlops:
    proj = core = mlp = 0.0
    for s in backbone.resolve():
        members = seq_len * s.k / s.G
        p = 8.0 * seq_len * s.dim * s.inner * s.k
        c = s.G * (2.0 if causal else 4.0) * members ** 2 * s.inner
        active = (s.k_p * s.h_pub + s.k * s.k_q * s.h_priv) if s.pool else (s.bank_top_k + s.dense_shared) * s.bank_width
        m = (6.0 if s.activation == "swiglu" else 4.0) * seq_len * s.dim * active     # three matrices gated, two pointwise
        proj += s.layers * p
        core += s.layers * c
        mlp += s.layers * m
    return BodyFlops(proj, core, mlp)


def body_flops(experiment: str, *, seq_len: int, causal: bool = True) -> BodyFlops:
    return backbone_body_flops(experiment_backbone(experiment), seq_len=seq_len, causal=causal)


def flops_per_token(experiment: str, *, seq_len: int, causal: bool = True) -> float:
    return body_flops(experiment, seq_len=seq_len, causal=causal).total / seq_len


def flop_ratio(experiment: str, reference: str, *, seq_len: int, causal: bool = True) -> float:
    return body_flops(experiment, seq_len=seq_len, causal=causal).total / body_flops(
        reference, seq_len=seq_len, causal=causal).total
