"""Evaluation: held-out language-modelling loss, routing statistics, long-context per-position loss."""

from nestor_b200.eval.suite import EvalSuite, LanguageModelingEval  # noqa: F401
from nestor_b200.eval.loading import load_experiment_checkpoint  # noqa: F401
from nestor_b200.eval.long_context import PerPositionLoss, sequence_nll, token_nll  # noqa: F401
