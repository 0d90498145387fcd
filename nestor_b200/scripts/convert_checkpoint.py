"""Rewrite a checkpoint's model weights between the two expert-bank layouts.

``--to per-expert`` turns the stacked banks (``stacked_public / stacked_private / stacked_moe_bank`` with
``w_up, w_gate [E, d, h]``, ``w_down [E, h, d]``) into one ``layers.0 / gate / layers.1`` weight set per expert
(``expert_pool.public_experts.{e}``, ``expert_pool.private_experts.{g}.{e}``, ``shared_experts.{e}``): the layout the
reference writes without ``NESTOR_STACKED_EXPERT_BANKS=1``. ``--to stacked`` is the inverse. The optimizer state is
indexed by parameter and therefore tied to a layout: it is dropped from the converted file (weights-only start, as
with ``DCLM_INIT_CHECKPOINT``). Loading either layout into this framework needs no conversion; the tool is for
moving weights the other way. Reference layouts: ``nestor/backbones/expert_bank_stack.py:58-213``,
``nestor/train/checkpoint.py:47-159``.
"""

from __future__ import annotations

import argparse
from pathlib import Path

import torch

from nestor_b200.train.checkpoint import is_stacked_state, stack_expert_banks, unstack_expert_banks


def private_experts_per_column(experiment: str) -> dict[str, int]:
    """``{layer prefix: Q}`` for every pooled layer of a registered experiment (the private bank is ``[G * Q, ...]``)."""

    from nestor_b200.experiments import discover_experiments, get_experiment
    discover_experiments()
    cfg = get_experiment(experiment)().jobs[0].model
    out = {}
    for b, s in enumerate(cfg.backbone_config.resolve()):
        if s.pool:
            for l in range(s.layers):
                out[f"backbone.blocks.{b}.layers.{l}"] = s.Q
    return out


def stacked_keys(experiment: str) -> set[str]:
    from nestor_b200.experiments import discover_experiments, get_experiment
    from nestor_b200.models import Model
    discover_experiments()
    with torch.device("meta"):
        return set(Model.from_config(get_experiment(experiment)().jobs[0].model).state_dict())


def convert(payload: dict, experiment: str, to: str) -> dict:
    key = "model" if "model" in payload else None
    state = payload[key] if key else payload
    if to == "per-expert":
        if not is_stacked_state(state):
            raise ValueError("the checkpoint already holds per-expert weights")
        new = unstack_expert_banks(state, private_experts_per_column(experiment))
    else:
        if is_stacked_state(state):
            raise ValueError("the checkpoint already holds stacked banks")
        new = stack_expert_banks(state, stacked_keys(experiment))
    if not key:
        return new
    out = {k: v for k, v in payload.items() if k not in ("optimizer", "scheduler")}
    out["model"] = new
    if payload.get("ema"):
        out["ema"] = (unstack_expert_banks(payload["ema"], private_experts_per_column(experiment)) if to == "per-expert"
                      else stack_expert_banks(payload["ema"], stacked_keys(experiment)))
    return out


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--experiment", required=True, help="registered experiment the checkpoint belongs to")
    ap.add_argument("--checkpoint", type=Path, required=True)
    ap.add_argument("--output", type=Path, required=True)
    ap.add_argument("--to", choices=("per-expert", "stacked"), required=True)
    a = ap.parse_args(argv)
    payload = torch.load(a.checkpoint, map_location="cpu", weights_only=False)
    out = convert(payload, a.experiment, a.to)
    a.output.parent.mkdir(parents=True, exist_ok=True)
    torch.save(out, a.output)
    n = len(out["model"] if "model" in out else out)
    print(f"wrote {a.output}: {n} tensors, {a.to} layout")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
