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
        valid = (aux or {}).get("valid_token_mask")
        if valid is not None:        # padded batch: padding positions are not targets
            target = target.masked_fill(~valid, PADDING_TOKEN_VALUE)
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


def _flat_router(router_aux: dict[str, Any]) -> tuple[Tensor, Tensor, Tensor]:
    """``(scores [N, C], topk_indices [N, k], valid [N])`` of one router record, tokens flattened."""

    scores = router_aux["scores"]
    C = scores.shape[-1]
    scores = scores.reshape(-1, C)
    idx = router_aux["topk_indices"].reshape(scores.shape[0], -1).long()
    valid = router_aux.get("valid_token_mask")
    valid = torch.ones(scores.shape[0], dtype=torch.bool, device=scores.device) if valid is None else valid.reshape(-1)
    return scores, idx, valid


def _assignment_counts(idx: Tensor, valid: Tensor, num_choices: int) -> Tensor:
    """How many valid tokens selected each choice (``[C]``, fp32, no gradient)."""

    w = valid.to(torch.float32).unsqueeze(-1).expand_as(idx).reshape(-1)
    return torch.zeros(num_choices, dtype=torch.float32, device=idx.device).scatter_add_(0, idx.reshape(-1), w)


def _router_records(aux: dict[str, Any] | None) -> tuple[list[dict], list[dict]]:
    """Group-router and expert-router records the backbone reported (``aux["blocks"][b]["group_router"]`` and
    ``aux["blocks"][b]["layers"][l]["expert_router"]``, each with ``scores`` and ``topk_indices``)."""

    groups, experts = [], []
    for block in (aux or {}).get("blocks", []):
        rec = block.get("group_router")
        if isinstance(rec, dict):
            groups.append(rec)
        for layer in block.get("layers", []):
            rec = layer.get("expert_router") if isinstance(layer, dict) else None
            if isinstance(rec, dict):
                experts.append(rec)
    return groups, experts


class RouterBalanceLoss(nn.Module):
    """Switch-style load-balance penalty, ``C * sum_c f_c p_c`` per router, with ``f`` the fraction of valid tokens
    assigned to choice ``c`` and ``p`` the mean softmax probability of ``c``; averaged over the group routers and,
    separately, over the expert routers (reference ``nestor/train/losses.py:288-400``)."""

    def __init__(self, config: RouterBalanceLossConfig) -> None:
        super().__init__()
        self.config = config

    @staticmethod
    def balance_term(router_aux: dict[str, Any]) -> Tensor:
        scores, idx, valid = _flat_router(router_aux)
        C = scores.shape[-1]
        vf = valid.to(torch.float32)
        n = vf.sum().clamp_min(1.0)
        assigned = _assignment_counts(idx, valid, C) / n
        routed = (torch.softmax(scores.float(), dim=-1) * vf.unsqueeze(-1)).sum(0) / n
        return C * (assigned * routed).sum()

    def forward(self, pred: Tensor, target: Tensor, aux: dict[str, Any] | None = None) -> LossOutput:
        groups, experts = _router_records(aux)
        total = pred.new_zeros((), dtype=torch.float32)
        comps: dict[str, Tensor] = {}
        for name, recs in (("router_balance_group", groups), ("router_balance_expert", experts)):
            if recs:
                term = torch.stack([self.balance_term(r) for r in recs]).mean() * self.config.balance_weight
                comps[name] = term.detach()
                total = total + term
        comps["router_balance"] = total.detach()
        return LossOutput(total=total, components=comps)


class ReferenceMoEAuxLoss(nn.Module):
    """Per-layer switch loss ``E * <normalize(sum probs), normalize(frequency)>`` with the assignment frequency
    summed over ranks, plus ``z_loss_weight * mean(logsumexp(scores)^2)``; summed over the layers' expert routers and
    scaled by ``coefficient`` (reference ``nestor/train/losses.py:403-486``)."""

    def __init__(self, config: ReferenceMoEAuxLossConfig) -> None:
        super().__init__()
        self.config = config

    def layer_term(self, router_aux: dict[str, Any]) -> Tensor:
        scores, idx, valid = _flat_router(router_aux)
        E = scores.shape[-1]
        logits = scores.float()
        vf = valid.to(torch.float32)
        acc_probs = (torch.softmax(logits, dim=-1) * vf.unsqueeze(-1)).sum(0)
        freq = _assignment_counts(idx, valid, E).detach()
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(freq)
        switch = E * (acc_probs / acc_probs.sum().clamp_min(1e-12) * (freq / freq.sum().clamp_min(1e-12))).sum()
        z = (torch.logsumexp(logits, dim=-1).square() * vf).sum() / vf.sum().clamp_min(1)
        return switch + self.config.z_loss_weight * z

    def forward(self, pred: Tensor, target: Tensor, aux: dict[str, Any] | None = None) -> LossOutput:
        _, experts = _router_records(aux)
        total = pred.new_zeros((), dtype=torch.float32)
        if experts:
            total = torch.stack([self.layer_term(r) for r in experts]).sum() * self.config.coefficient
        return LossOutput(total=total, components={"reference_moe_aux": total.detach()})


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
