"""Rank-0 console logging with optional wandb mirroring (reference: ``nestor/utils/logging.py:41-78``)."""

from __future__ import annotations

import logging
import sys
from typing import Any, Mapping

from nestor_b200.utils.distributed import is_main_process

_wandb_run = None


def get_logger(name: str = "nestor_b200") -> logging.Logger:
    logger = logging.getLogger(name)
    if not logger.handlers:
        h = logging.StreamHandler(sys.stdout)
        h.setFormatter(logging.Formatter("%(asctime)s %(name)s %(levelname)s %(message)s", "%H:%M:%S"))
        logger.addHandler(h)
        logger.propagate = False
    logger.setLevel(logging.INFO if is_main_process() else logging.WARNING)
    return logger


def set_wandb_run(run: Any) -> None:
    global _wandb_run
    _wandb_run = run


def log_metrics(logger: logging.Logger, metrics: Mapping[str, Any], step: int, prefix: str = "") -> None:
    """Print ``key=value`` pairs on rank 0 and mirror them to wandb when a run is active."""

    if not is_main_process():
        return
    parts = []
    for k, v in metrics.items():
        parts.append(f"{k}={v:.5g}" if isinstance(v, float) else f"{k}={v}")
    logger.info("step %d | %s", step, " ".join(parts))
    if _wandb_run is not None:
        _wandb_run.log({f"{prefix}{k}": v for k, v in metrics.items()}, step=step)
