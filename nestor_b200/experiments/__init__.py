"""Experiment registry and the registered pretraining cells."""

from nestor_b200.experiments.registry import (  # noqa: F401
    get_experiment, list_experiments, register_experiment, discover_experiments,
)
