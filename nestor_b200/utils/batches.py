"""Unpacking of supervised batches (same accepted forms as the reference's ``nestor/utils/batches.py:11-63``)."""

from __future__ import annotations

from collections.abc import Mapping
from typing import Any

from torch import Tensor

_PAIRS = (("inputs", "targets"), ("inputs", "labels"), ("x", "y"))


def split_supervised_batch(batch: Any) -> tuple[Any, Tensor]:
    """``(model inputs, targets)`` from a 2-tuple / 2-list, or from a mapping with ``inputs``/``targets``,
    ``inputs``/``labels`` or ``x``/``y``. Targets must be a tensor; anything else is a ``TypeError``."""

    if isinstance(batch, (tuple, list)) and len(batch) == 2:
        inputs, targets = batch
    elif isinstance(batch, Mapping):
        for a, b in _PAIRS:
            if a in batch and b in batch:
                inputs, targets = batch[a], batch[b]
                break
        else:
            raise TypeError(f"Unsupported supervised batch keys {sorted(map(str, batch))}; expected one of "
                            + ", ".join(f"{a}/{b}" for a, b in _PAIRS) + ".")
    else:
        raise TypeError(f"Unsupported supervised batch of type {type(batch).__name__}; expected an (inputs, targets) "
                        "pair or a mapping.")
    if not isinstance(targets, Tensor):
        raise TypeError(f"Expected supervised targets to be a Tensor, got {type(targets).__name__}.")
    return inputs, targets
