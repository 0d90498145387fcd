"""Describe a registered experiment without running it: block geometry, parameter counts by optimizer, FLOPs per token,
tokens per step, and the per-GPU footprint of the parameter arenas and the optimizer state at a given world size.

``python -m nestor_b200.scripts.describe --experiment nestor_200m [--world 8] [--json]``. The model is instantiated
on the ``meta`` device (no memory is allocated), so this also answers "does this configuration resolve" for a
hand-edited experiment in seconds on a login node.
"""

from __future__ import annotations

import argparse
import json
from typing import Any

import torch


def describe(experiment: str, world: int = 1) -> dict[str, Any]:
    from nestor_b200.experiments import discover_experiments, get_experiment
    from nestor_b200.models import Model
    from nestor_b200.models.tags import get_tag
    from nestor_b200.train.flops import forward_flops_per_token, train_flops_per_token

    discover_experiments()
    job = get_experiment(experiment)().jobs[0]
    cfg = job.model
    with torch.device("meta"):
        model = Model.from_config(cfg)
    by_optimizer: dict[str, int] = {}
    trainable = frozen = 0
    for p in model.parameters():
        if not p.requires_grad:
            frozen += p.numel()
            continue
        trainable += p.numel()
        name = get_tag(p).optimizer
        by_optimizer[name] = by_optimizer.get(name, 0) + p.numel()
    seq = int(getattr(job.train_dataset, "block_size", 0) or 0)
    batch = int(getattr(job.train_dataloader, "batch_size", 0) or 0)
    accum = int(job.grad_accum_steps)
    blocks = []
    for s in cfg.backbone_config.resolve():
        row: dict[str, Any] = {"block": s.index, "layers": s.layers, "columns": s.G, "columns_per_token": s.k,
                               "heads": s.heads, "head_dim": s.head_dim, "exports": s.exports if cfg.backbone_config.column_mode else 1}
        if s.pool:
            row["experts"] = f"pool: {s.P} public (top {s.k_p}, width {s.h_pub}) + {s.Q} private per column (top {s.k_q}, width {s.h_priv})"
        else:
            sizes = s.layer_experts or (s.bank_experts,)
            row["experts"] = (f"bank: {'/'.join(map(str, sizes))} experts (top {s.bank_top_k}, width {s.bank_width}, "
                              f"{s.activation})" if max(sizes) > 1 else f"dense MLP (width {s.bank_width}, {s.activation})")
        blocks.append(row)
    gib = 2.0 ** 30
    # fp32 master + fp32 gradient + bf16 compute copy are replicated; Muon keeps one fp32 momentum, AdamW two fp32
    # moments, both sharded over the ranks' arena ranges (ZeRO-1)
    arenas = trainable * (4 + 4 + 2) / gib
    state = (by_optimizer.get("muon", 0) * 4 + sum(v for k, v in by_optimizer.items() if k != "muon") * 8) / gib
    return {
        "experiment": experiment, "residual_topology": cfg.backbone_config.block_residual_mode,
        "causal": bool(cfg.backbone_config.causal), "width": cfg.backbone_config.input_dim, "blocks": blocks,
        "parameters": {"total": trainable + frozen, "trainable": trainable, "frozen": frozen, "by_optimizer": by_optimizer},
        "sequence_length": seq, "tokens_per_step": seq * batch * accum,
        "flops_per_token": {"forward": forward_flops_per_token(cfg, seq), "training": train_flops_per_token(cfg, seq)},
        "per_gpu_gib": {"world": world, "parameter_arenas": round(arenas, 2),
                        "optimizer_state": round(state / max(world, 1), 2)},
    }


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--experiment", required=True)
    ap.add_argument("--world", type=int, default=1, help="ranks the optimizer state is sharded over")
    ap.add_argument("--json", action="store_true")
    a = ap.parse_args(argv)
    info = describe(a.experiment, a.world)
    if a.json:
        print(json.dumps(info, indent=2))
        return 0
    p = info["parameters"]
    print(f"{info['experiment']}: width {info['width']}, {info['residual_topology']}, "
          f"{'causal' if info['causal'] else 'bidirectional'}, sequence {info['sequence_length']}, "
          f"{info['tokens_per_step']:,} tokens per optimizer step")
    for b in info["blocks"]:
        print(f"  block {b['block']}: {b['layers']} layers, {b['columns_per_token']} of {b['columns']} columns, "
              f"{b['heads']} heads x {b['head_dim']}, {b['exports']} depth source(s); {b['experts']}")
    print(f"  parameters: {p['total']:,} ({p['trainable']:,} trainable; " +
          ", ".join(f"{k} {v:,}" for k, v in sorted(p["by_optimizer"].items())) + ")")
    f = info["flops_per_token"]
    print(f"  FLOPs per token: forward {f['forward']:.4g}, training {f['training']:.4g}")
    g = info["per_gpu_gib"]
    print(f"  per GPU at world {g['world']}: parameter arenas {g['parameter_arenas']} GiB, optimizer state {g['optimizer_state']} GiB")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
