"""Name -> experiment-function registry.

An experiment is a zero-argument function returning an ``ExperimentConfig``; its
``__name__`` is the name ``nestor_cli --experiment`` takes. Behavioural parity with
``nestor/experiments/registry.py:19-76`` of the reference: duplicate names raise
``ValueError``, unknown names raise ``KeyError`` listing what exists, listing is sorted.
"""

from __future__ import annotations

import importlib
import pkgutil
from typing import Callable

_CELLS: dict[str, Callable[[], object]] = {}


def register_experiment(fn: Callable[[], object]) -> Callable[[], object]:
    name = getattr(fn, "__name__", None)
    if not isinstance(name, str):
        raise TypeError("register_experiment needs a named function.")
    if name in _CELLS:
        raise ValueError(f"Experiment '{name}' is already registered.")
    _CELLS[name] = fn
    return fn


def get_experiment(name: str) -> Callable[[], object]:
    try:
        return _CELLS[name]
    except KeyError:
        known = ", ".join(sorted(_CELLS)) or "(none)"
        raise KeyError(f"Experiment '{name}' not found. Available: {known}") from None


def list_experiments() -> list[str]:
    return sorted(_CELLS)


def discover_experiments() -> None:
    """Import every module of this package so their ``@register_experiment`` calls run."""

    import nestor_b200.experiments as pkg

    for info in pkgutil.iter_modules(pkg.__path__):
        if info.name != "registry":
            importlib.import_module(f"{pkg.__name__}.{info.name}")
