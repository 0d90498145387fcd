"""FLOP accounting for MFU metrics.

Two counts of the same thing. The analytic one (body FLOPs from :mod:`nestor_b200.continual.flops` + routers + LM
head, times three for forward+backward) is what the trainer uses every step: the matrix products run in custom
kernels that ``FlopCounterMode`` cannot see. The measured one (:func:`calibrate_flops`) runs the PyTorch statement of
the model once under ``FlopCounterMode`` on a short sequence, where every product is an ``aten`` matmul the counter
knows, and reports how far the analytic formula is from it; ``NESTOR_MFU_CALIBRATE=1`` makes the trainer log that
ratio and scale its numerator by it. Reference: ``nestor/train/trainer.py:582-758`` (calibration),
``nestor/train/flop_formulas.py:30-91`` (grouped-GEMM formula).
"""

from __future__ import annotations

import copy
from typing import Any

import torch

from nestor_b200.configs.model import SequenceModelConfig
from nestor_b200.continual.flops import backbone_body_flops

_REGISTERED = False


def register_extra_flop_formulas() -> bool:
    """Teach ``FlopCounterMode`` the grouped GEMM (``aten._grouped_mm``): ``2 * rows * K * N`` whatever the grouping.
    Idempotent and never raises (a torch without the op or with another registration API leaves it uncounted)."""

    global _REGISTERED
    if _REGISTERED:
        return True
    try:
        from torch.utils.flop_counter import register_flop_formula
        op = getattr(torch.ops.aten, "_grouped_mm", None)
        if op is None:
            return False

        def formula(a_shape, b_shape, *args: Any, out_shape=None, **kwargs: Any) -> int:
            rows = 1
            for dim in a_shape[:-1]:
                rows *= int(dim)
            return grouped_mm_flops(rows, int(a_shape[-1]), int(b_shape[-1]))

        register_flop_formula(op)(formula)
        _REGISTERED = True
    except Exception:  # noqa: BLE001 - MFU accounting must never break training
        return False
    return True


@torch.no_grad()
def calibrate_flops(model: Any, seq_len: int = 128, batch: int = 1) -> dict[str, float]:
    """Count the forward FLOPs of ``model`` on ``[batch, seq_len]`` tokens with ``FlopCounterMode`` (CPU copy, PyTorch
    statement of every op) and compare with the analytic formula at the same length.

    Returns ``{"counted", "analytic", "ratio"}`` in forward FLOPs per token. The counter sees matrix products only,
    which is also all the analytic formula claims to count.
    """

    from torch.utils.flop_counter import FlopCounterMode
    from nestor_b200 import ops
    register_extra_flop_formulas()
    twin = copy.deepcopy(model).to("cpu").float().eval()
    for mod in twin.modules():                       # a CPU twin reads its own parameters, not a GPU arena's views
        mod.__dict__.pop("_nestor_arena", None)
    twin.compute_dtype, twin.fused_head = torch.float32, False
    vocab = twin.head.vocab_size
    ids = torch.randint(0, vocab, (batch, seq_len))
    with ops.oracle_ops(), FlopCounterMode(display=False) as counter:
        twin(ids)
    counted = counter.get_total_flops() / (batch * seq_len)
    analytic = forward_flops_per_token(model.config, seq_len)
    return {"counted": counted, "analytic": analytic, "ratio": counted / analytic}


def grouped_mm_flops(rows: int, k: int, n: int) -> int:
    """FLOPs of a grouped GEMM over ``rows`` total rows: ``2 * rows * K * N`` (group count is irrelevant)."""

    return 2 * rows * k * n


def forward_flops_per_token(config: SequenceModelConfig, seq_len: int) -> float:
    bb = config.backbone_config
    body = backbone_body_flops(bb, seq_len=seq_len, causal=bool(getattr(bb, "causal", True))).total / seq_len
    routers = 0.0
    for s in bb.resolve():
        if s.G > 1:
            routers += 2 * 2.0 * (s.dim * s.router_hidden + s.router_hidden * s.G)   # score + noise MLPs, once per block
        if s.pool:
            routers += s.layers * 2.0 * s.dim * (s.P + s.G * s.Q + 2)
        else:
            routers += sum(2.0 * s.dim * s.experts_of_layer(i) for i in range(s.layers))
    head = 2.0 * bb.output_dim * config.head_config.vocab_size
    return body + routers + head


def train_flops_per_token(config: SequenceModelConfig, seq_len: int) -> float:
    return 3.0 * forward_flops_per_token(config, seq_len)
