"""FLOP accounting for MFU metrics.

The reference calibrates with ``FlopCounterMode`` on a small batch and patches in a
formula for grouped GEMMs (``nestor/train/trainer.py:582-758``, ``train/flop_formulas.py:30-91``).
Every matrix product here runs in a custom kernel the counter cannot see, so the count is
analytic: body FLOPs from :mod:`nestor_b200.continual.flops` + routers + LM head,
times three for forward+backward.
"""

from __future__ import annotations

from nestor_b200.configs.model import SequenceModelConfig
from nestor_b200.continual.flops import backbone_body_flops


def grouped_mm_flops(rows: int, k: int, n: int) -> int:
    """FLOPs of a grouped GEMM over ``rows`` total rows: ``2 * rows * K * N`` (group count is irrelevant)."""

    return 2 * rows * k * n


def forward_flops_per_token(config: SequenceModelConfig, seq_len: int) -> float:
    bb = config.backbone_config
    body = backbone_body_flops(bb, seq_len=seq_len).total / seq_len
    routers = 0.0
    for s in bb.resolve():
        if s.G > 1:
            routers += 2 * 2.0 * (s.dim * s.router_hidden + s.router_hidden * s.G)   # score + noise MLPs, once per block
        per_layer = (2.0 * s.dim * (s.P + s.G * s.Q + 2)) if s.pool else 2.0 * s.dim * s.bank_experts
        routers += s.layers * per_layer
    head = 2.0 * bb.output_dim * config.head_config.vocab_size
    return body + routers + head


def train_flops_per_token(config: SequenceModelConfig, seq_len: int) -> float:
    return 3.0 * forward_flops_per_token(config, seq_len)
