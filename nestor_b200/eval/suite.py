"""Evaluation suite: held-out cross-entropy / perplexity plus routing statistics, summed over ranks.

``EvalSuite(config, device).run(model)`` evaluates every configured eval and returns
``{eval_name: {metric: value}}``. ``LanguageModelingEval`` walks its dataset in rank-strided order
(padded so every rank runs the same number of batches, padded rows masked out), sums loss and token
counts across ranks and reports ``cross_entropy`` and ``perplexity`` with per-router routing
metrics. Reference: ``nestor/eval/suite.py:50-278``.
"""

from __future__ import annotations

import math
from typing import Any

import torch

from nestor_b200 import ops
from nestor_b200.configs import EvalConfig, EvalSuiteConfig, LanguageModelingEvalConfig
from nestor_b200.data.datasets import build_dataset
from nestor_b200.eval.metrics import routing_metrics
from nestor_b200.models.nestor import router_counts, router_prob_sums
from nestor_b200.train.losses import ce_chunk_rows
from nestor_b200.utils.distributed import get_padded_rank_indices, get_rank, get_world_size, sum_tensor_across_ranks


class LanguageModelingEval:
    def __init__(self, config: LanguageModelingEvalConfig, device: torch.device) -> None:
        self.config, self.device = config, device
        self.dataset = build_dataset(config.dataset_config)
        self.batch_size = max(1, config.dataloader_config.batch_size // max(1, get_world_size()))

    @torch.no_grad()
    def run(self, model: Any) -> dict[str, Any]:
        was_training, was_fused = model.training, model.fused_head
        model.eval()
        # the head runs inside the chunked head + cross-entropy op: no [B, S, V] logits tensor ever exists (at most
        # NESTOR_CE_CHUNK_ROWS x V at a time; the reference chunks its evaluation head too, nestor/eval/long_context.py:75)
        model.fused_head = True
        head = model.head
        n = len(self.dataset)
        idx = get_padded_rank_indices(n)
        real = set(range(n)[get_rank()::get_world_size()])
        totals = torch.zeros(2, dtype=torch.float64, device=self.device)
        counts: dict[str, torch.Tensor] = {}
        probs: dict[str, torch.Tensor] = {}
        for a in range(0, len(idx), self.batch_size):
            rows = idx[a : a + self.batch_size]
            ids = torch.stack([self.dataset[i][0] for i in rows]).to(self.device)
            keep = torch.tensor([i in real for i in rows], device=self.device)
            out = model(ids)
            hidden = out.pred[:, :-1].reshape(-1, out.pred.shape[-1])
            targets = ids[:, 1:].masked_fill(~keep.unsqueeze(1), -100).reshape(-1)     # padded rows are not targets
            nll_sum, n_targets = ops.lm_head_ce(hidden, head.weight, targets, head.logit_multiplier, hidden.dtype,
                                                chunk_rows=ce_chunk_rows())
            totals[0] += nll_sum.double()
            totals[1] += n_targets.double()
            if bool(keep.all()):
                for k, v in router_counts(model.backbone, out.aux).items():
                    counts[k] = v if k not in counts else counts[k] + v
                for k, v in router_prob_sums(model.backbone, out.aux).items():
                    probs[k] = v if k not in probs else probs[k] + v
        sum_tensor_across_ranks(totals)
        for k in sorted(counts):
            sum_tensor_across_ranks(counts[k])
        for k in sorted(probs):
            sum_tensor_across_ranks(probs[k])
        ce = float(totals[0] / totals[1].clamp_min(1))
        model.fused_head = was_fused
        model.train(was_training)
        result = {"cross_entropy": ce, "perplexity": math.exp(min(ce, 50.0)), "tokens": int(totals[1].item())}
        result.update(routing_metrics({k: v.cpu() for k, v in counts.items()}, {k: v.cpu() for k, v in probs.items()}))
        return result


def build_eval(config: EvalConfig, device: torch.device) -> Any:
    if isinstance(config, LanguageModelingEvalConfig):
        return LanguageModelingEval(config, device)
    raise TypeError(f"Unknown eval config {type(config).__name__}.")


class EvalSuite:
    def __init__(self, config: EvalSuiteConfig, device: torch.device) -> None:
        self.evals = [(c.name, build_eval(c, device)) for c in config.evals]

    @classmethod
    def from_config(cls, config: EvalSuiteConfig, device: torch.device) -> "EvalSuite":
        return cls(config, device)

    def run(self, model: Any) -> dict[str, dict[str, Any]]:
        return {name: ev.run(model) for name, ev in self.evals}
