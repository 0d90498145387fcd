"""Training losses.

``CausalLMLoss`` is the mean shifted cross-entropy over valid targets (reference
``nestor/train/losses.py:122-285``). With a fused head (``aux["fused_head_module"]``) it
runs the chunked head+CE op, which never materialises ``[T, V]`` logits; otherwise it
takes logits. ``RouterBalanceLoss`` and ``ReferenceMoEAuxLoss`` are the optional
auxiliary recipes (``:288-486``); ``CompositeLoss`` sums weighted parts.
"""

from __future__ import annotations

import dataclasses as dc
import os
from typing import Any

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch import Tensor, nn
from torch.utils.checkpoint import checkpoint

from nestor_b200 import ops
from nestor_b200.configs import (
    CausalLMLossConfig, CompositeLossConfig, LossConfig, ReferenceMoEAuxLossConfig, RouterBalanceLossConfig,
)
from nestor_b200.constants import PADDING_TOKEN_VALUE


@dc.dataclass
class LossOutput:
    total: Tensor
    components: dict[str, Tensor]


def ce_chunk_rows() -> int:
    return int(os.environ.get("NESTOR_CE_CHUNK_ROWS", "0")) or 4096


class CausalLMLoss(nn.Module):
    def __init__(self, config: CausalLMLossConfig | None = None) -> None:
        super().__init__()
        self.config = config or CausalLMLossConfig()

    @staticmethod
    def sum_loss_and_tokens(pred: Tensor, target: Tensor, *, valid_token_mask: Tensor | None = None,
                            ignore_index: int = PADDING_TOKEN_VALUE, label_smoothing: float = 0.0,
                            chunk_rows: int = 0) -> tuple[Tensor, Tensor]:
        """Summed CE of logits ``pred [B, S, V]`` against next tokens; optional row-chunked recompute."""

        logits = pred[:, :-1, :].reshape(-1, pred.shape[-1])
        tgt = target[:, 1:].reshape(-1)
        if valid_token_mask is not None:
            if valid_token_mask.shape != target[:, 1:].shape:
                raise ValueError("valid_token_mask must match target[:, 1:].")
            tgt = tgt.masked_fill(~valid_token_mask.reshape(-1), ignore_index)
        count = (tgt != ignore_index).sum()

        def ce(lg: Tensor, tg: Tensor) -> Tensor:
            return F.cross_entropy(lg.float(), tg, ignore_index=ignore_index,
                                   label_smoothing=label_smoothing, reduction="sum")

        if chunk_rows > 0 and logits.requires_grad:
            total = logits.new_zeros((), dtype=torch.float32)
            for a in range(0, logits.shape[0], chunk_rows):
                total = total + checkpoint(ce, logits[a : a + chunk_rows], tgt[a : a + chunk_rows],
                                           use_reentrant=False)
            return total, count
        return ce(logits, tgt), count

    def forward(self, pred: Tensor, target: Tensor, aux: dict[str, Any] | None = None) -> LossOutput:
        head = (aux or {}).get("fused_head_module")
        if head is not None:
            hidden = pred[:, :-1, :].reshape(-1, pred.shape[-1])
            tgt = target[:, 1:].reshape(-1)
            if self.config.label_smoothing:
                raise ValueError("label smoothing is not available with the fused head+CE path.")
            cd = hidden.dtype
            loss_sum, count = ops.lm_head_ce(hidden, head.weight, tgt, head.logit_multiplier, cd,
                                             chunk_rows=ce_chunk_rows())
        else:
            loss_sum, count = self.sum_loss_and_tokens(
                pred, target, label_smoothing=self.config.label_smoothing,
                chunk_rows=int(os.environ.get("NESTOR_CE_CHUNK_ROWS", "0")))
        loss = loss_sum / count.clamp_min(1).to(loss_sum.dtype)
        return LossOutput(total=loss, components={"cross_entropy": loss, "perplexity": loss.detach().exp()})


def _router_stats(aux: dict[str, Any]) -> list[tuple[Tensor, int]]:
    """(indices, num_choices) for every router that reported its selection."""

    out = []
    for block in (aux or {}).get("blocks", []):
        gi = block.get("group_idx")
        if gi is not None and block.get("num_groups", 0) > 1:
            out.append((gi, block["num_groups"]))
    return out


class RouterBalanceLoss(nn.Module):
    """Switch-style load-balance penalty on the group routers' hard assignment fractions."""

    def __init__(self, config: RouterBalanceLossConfig) -> None:
        super().__init__()
        self.config = config

    def forward(self, pred: Tensor, target: Tensor, aux: dict[str, Any] | None = None) -> LossOutput:
        terms = []
        for idx, n in _router_stats(aux or {}):
            frac = torch.bincount(idx.reshape(-1), minlength=n).float()
            frac = frac / frac.sum().clamp_min(1)
            terms.append(n * (frac * frac).sum() - 1.0)
        total = pred.new_zeros((), dtype=torch.float32)
        if terms:
            total = self.config.balance_weight * torch.stack(terms).mean()
        return LossOutput(total=total, components={"router_balance": total.detach()})


class ReferenceMoEAuxLoss(nn.Module):
    """``coefficient * E * sum_e f_e p_e`` with ``f`` summed across ranks, plus a router z-loss."""

    def __init__(self, config: ReferenceMoEAuxLossConfig) -> None:
        super().__init__()
        self.config = config

    def forward(self, pred: Tensor, target: Tensor, aux: dict[str, Any] | None = None) -> LossOutput:
        total = pred.new_zeros((), dtype=torch.float32)
        for rec in (aux or {}).get("moe_aux", []):
            probs, idx = rec["probs"], rec["idx"]
            E = probs.shape[-1]
            freq = torch.bincount(idx.reshape(-1), minlength=E).float()
            if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
                dist.all_reduce(freq)
            freq = freq / freq.sum().clamp_min(1)
            total = total + self.config.coefficient * E * (freq * probs.float().mean(dim=0)).sum()
            total = total + self.config.z_loss_weight * torch.logsumexp(rec["scores"].float(), dim=-1).pow(2).mean()
        return LossOutput(total=total, components={"moe_aux": total.detach()})


class CompositeLoss(nn.Module):
    def __init__(self, config: CompositeLossConfig) -> None:
        super().__init__()
        self.parts = nn.ModuleList([build_loss(c) for c in config.losses])
        self.weights = list(config.weights) or [1.0] * len(self.parts)

    def forward(self, pred: Tensor, target: Tensor, aux: dict[str, Any] | None = None) -> LossOutput:
        total, comps = None, {}
        for w, part in zip(self.weights, self.parts):
            out = part(pred, target, aux)
            total = w * out.total if total is None else total + w * out.total
            comps.update(out.components)
        return LossOutput(total=total, components=comps)


def build_loss(config: LossConfig) -> nn.Module:
    if isinstance(config, CausalLMLossConfig):
        return CausalLMLoss(config)
    if isinstance(config, RouterBalanceLossConfig):
        return RouterBalanceLoss(config)
    if isinstance(config, ReferenceMoEAuxLossConfig):
        return ReferenceMoEAuxLoss(config)
    if isinstance(config, CompositeLossConfig):
        return CompositeLoss(config)
    raise TypeError(f"Unknown loss config {type(config).__name__}.")
