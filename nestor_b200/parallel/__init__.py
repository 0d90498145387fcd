"""Data-parallel machinery: parameter arena, gradient reduction, sharded-optimizer sync, symmetric memory."""

from nestor_b200.parallel.arena import ParamArena, arena_of  # noqa: F401
