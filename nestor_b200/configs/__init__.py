"""Keyword-only dataclass configs (the config-first API surface).

Field names follow the reference's ``nestor/configs/*.py`` so experiment functions
written against either stack construct the same objects; the classes are grouped
into two modules here (``run`` for jobs/data/optim/sched/loss, ``model`` for the
model composition).
"""

from nestor_b200.configs.run import *  # noqa: F401,F403
from nestor_b200.configs.model import *  # noqa: F401,F403
