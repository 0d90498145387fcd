"""Run orchestration: run directories, config/git sidecars, resume, train and eval pipelines."""

from nestor_b200.pipelines.run import (  # noqa: F401
    EvalPipeline, RunContext, TrainPipeline, find_latest_checkpoint, resolve_resume_checkpoint,
)
