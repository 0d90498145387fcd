"""Rebuild a registered model from a checkpoint for evaluation.

The expert-bank layout of the file is detected from its keys (stacked banks carry
``.stacked_`` keys) and converted on load; the load is by name and shape and refuses to leave any
model parameter uninitialised. Reference: ``nestor/eval/checkpoint.py:25-100``.
"""

from __future__ import annotations

from pathlib import Path
from typing import Any

import torch

from nestor_b200.experiments import discover_experiments, get_experiment
from nestor_b200.models import Model
from nestor_b200.train.checkpoint import is_stacked_state, load_init_state


def load_experiment_checkpoint(experiment: str, checkpoint: Path, device: torch.device | str = "cpu",
                               dtype: torch.dtype = torch.float32, use_ema: bool = False) -> tuple[Any, dict]:
    """Returns ``(model in eval mode, info)``; ``info`` reports the step, layout and skipped keys."""

    discover_experiments()
    job = get_experiment(experiment)().jobs[0]
    model = Model.from_config(job.model)
    ckpt = torch.load(checkpoint, map_location="cpu", weights_only=False)
    state = ckpt.get("ema") if use_ema and ckpt.get("ema") else ckpt.get("model", ckpt)
    loaded, skipped = load_init_state(model, state, allow_partial=False)
    model.to(device=device)
    model.compute_dtype = dtype if torch.device(device).type == "cuda" or dtype == torch.float32 else torch.float32
    model.eval()
    return model, {"step": ckpt.get("step"), "stacked": is_stacked_state(state), "loaded": loaded,
                   "skipped": sorted(skipped), "git_sha": ckpt.get("git_sha")}
