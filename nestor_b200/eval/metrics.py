"""Routing statistics from selection counts.

``routing_metrics`` turns per-router selection counts (``router_counts`` of the backbone, summed
over an evaluation and over ranks) into the flat metric names the reference logs
(``nestor/eval/metrics.py:197-270``): per-choice assignment fractions, the largest fraction, and a
balance score ``1 - cv / cv_max`` (1 = perfectly even, 0 = everything on one choice), plus
per-kind means. The ``prob/*`` entries (mean softmax routing mass per choice) come from the probability
sums the model attaches to evaluation forwards (``models.nestor.router_prob_sums``).
"""

from __future__ import annotations

import math

import torch
from torch import Tensor


def router_entropy(probs: Tensor) -> Tensor:
    """Mean entropy (nats) of routing distributions ``[..., choices]``."""

    p = probs.float().clamp_min(1e-10)
    return -(p * p.log()).sum(dim=-1).mean()


def load_balance(counts: Tensor) -> float:
    n = counts.numel()
    if n < 2:
        return 1.0
    load = counts.float() / counts.float().sum().clamp_min(1.0)
    cv = float(load.std(unbiased=False) / load.mean().clamp_min(1e-10))
    return max(0.0, 1.0 - cv / math.sqrt((n - 1) / n))


def router_kind(name: str) -> str:
    if name.endswith("group_router"):
        return "group"
    if "private_routers" in name:
        return "private"
    if name.endswith("public_router"):
        return "public"
    return "expert"


def routing_metrics(counts: dict[str, Tensor], prob_sums: dict[str, Tensor] | None = None) -> dict[str, float]:
    out: dict[str, float] = {}
    by_kind: dict[str, dict[str, list[float]]] = {}
    for name, c in sorted(counts.items()):
        total = float(c.sum())
        if total <= 0 or c.numel() < 2:
            continue
        frac = (c.float() / total).tolist()
        for i, f in enumerate(frac):
            out[f"routing/{name}/frac/c{i}"] = float(f)
        out[f"routing/{name}/max_frac"] = max(frac)
        bal = load_balance(c)
        out[f"routing/{name}/balance"] = bal
        k = by_kind.setdefault(router_kind(name), {"balance": [], "max_frac": [], "max_prob": []})
        k["balance"].append(bal)
        k["max_frac"].append(max(frac))
        if prob_sums and name in prob_sums:
            pr = (prob_sums[name].float() / prob_sums[name].float().sum().clamp_min(1e-10)).tolist()
            for i, p in enumerate(pr):
                out[f"routing/{name}/prob/c{i}"] = float(p)
            out[f"routing/{name}/max_prob"] = max(pr)
            k["max_prob"].append(max(pr))
    for kind, vals in by_kind.items():
        for key, xs in vals.items():
            if xs:
                out[f"routing/{kind}/mean_{key}"] = sum(xs) / len(xs)
    return out
