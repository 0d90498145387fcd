"""Seeding and numeric-mode switches (reference: ``nestor/utils/seed.py:11-31``)."""

from __future__ import annotations

import os
import random

import numpy as np
import torch


def set_seed(seed: int, *, rank_offset: int = 0) -> None:
    """Seed python / numpy / torch; TF32 'high' matmul precision; optional determinism.

    ``NESTOR_DETERMINISTIC=1`` turns on cuDNN determinism and disables autotuning.
    """

    s = int(seed) + int(rank_offset)
    random.seed(s)
    np.random.seed(s % (2**32))
    torch.manual_seed(s)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(s)
    torch.set_float32_matmul_precision("high")
    if os.environ.get("NESTOR_DETERMINISTIC") == "1":
        torch.backends.cudnn.deterministic = True
        torch.backends.cudnn.benchmark = False
    else:
        torch.backends.cudnn.benchmark = True
