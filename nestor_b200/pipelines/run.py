"""Train / eval pipelines.

A pipeline owns one job of an experiment: it joins the process group, seeds, creates
``<output_root>/<experiment>/<timestamp>__<job>/`` with ``config.json`` and ``git_sha.txt``,
optionally starts (or continues) a wandb run, builds data / model / trainer and runs.
Resume policy (reference ``nestor/pipelines/train.py:23-92``, ``157-194``): an explicit strict
checkpoint wins; otherwise the newest ``model_<step>.pt`` under any earlier run directory of
the same experiment is resumed strictly; otherwise an explicit non-strict checkpoint only
initialises weights; otherwise training starts fresh.
"""

from __future__ import annotations

import json
import os
from datetime import datetime
from pathlib import Path
from typing import Any

import torch

from nestor_b200.configs import EvalJobConfig, ExperimentConfig, TrainJobConfig, config_to_dict
from nestor_b200.data.datasets import PinnedWindowLoader, build_dataset
from nestor_b200.models import Model
from nestor_b200.train.checkpoint import get_git_sha
from nestor_b200.train.trainer import Trainer
from nestor_b200.utils import logging as nlog
from nestor_b200.utils.distributed import barrier, get_rank, get_world_size, init_distributed, is_main_process
from nestor_b200.utils.seed import set_seed


def find_latest_checkpoint(experiment_dir: Path, *, exclude_run_dir: Path | None = None,
                           checkpoint_dir: Path | str = "checkpoints") -> tuple[Path | None, int]:
    best, best_step = None, -1
    root = Path(experiment_dir)
    if not root.exists():
        return None, -1
    for run in root.iterdir():
        if not run.is_dir() or run == exclude_run_dir:
            continue
        for f in (run / checkpoint_dir).glob("model_[0-9]*.pt"):
            try:
                step = int(f.stem.split("_", 1)[1])
            except (IndexError, ValueError):
                continue
            if step > best_step:
                best, best_step = f, step
    return best, best_step


def resolve_resume_checkpoint(*, explicit: Path | None, explicit_strict: bool,
                              latest_own: Path | None) -> tuple[Path | None, bool, str]:
    if explicit is not None and explicit_strict:
        return explicit, True, "explicit"
    if latest_own is not None:
        return latest_own, True, "auto"
    if explicit is not None:
        return explicit, False, "init"
    return None, True, "none"


class RunContext:
    """Process group, seed, run directory and sidecar files of one job."""

    def __init__(self, job: Any, experiment: ExperimentConfig) -> None:
        self.job, self.experiment = job, experiment
        self.device = init_distributed(enabled=job.distributed.enabled)
        self.logger = nlog.get_logger("nestor_b200")
        set_seed(job.seed if job.seed is not None else 42)
        stamp = [datetime.now().strftime("%Y%m%d_%H%M%S")]
        if get_world_size() > 1:  # every rank must agree on the directory name
            torch.distributed.broadcast_object_list(stamp, src=0)
        self.run_dir = Path(experiment.output_root) / experiment.name / f"{stamp[0]}__{job.name}"
        if is_main_process():
            self.run_dir.mkdir(parents=True, exist_ok=True)
            (self.run_dir / "config.json").write_text(json.dumps(
                {"experiment": config_to_dict(experiment), "job": config_to_dict(job)}, indent=2, default=str))
            sha = get_git_sha()
            if sha:
                (self.run_dir / "git_sha.txt").write_text(sha + "\n")
            if getattr(experiment, "save_source_snapshot", False):
                from nestor_b200.utils.snapshot import snapshot_sources
                repo = Path(__file__).resolve().parents[2]
                snapshot_sources(repo, self.run_dir / "source_snapshot.zip")
            self.logger.info("Run directory: %s", self.run_dir)
        barrier()
        self.wandb_run = None

    def init_wandb(self, resume_from: Path | None = None) -> None:
        """Start a wandb run on rank 0 unless disabled; continue the id stored beside a resumed run."""

        job = self.job
        if not is_main_process() or not getattr(job, "wandb_project", None):
            return
        if os.environ.get("WANDB_MODE", "").lower() in ("disabled", "offline-skip"):
            return
        try:
            import wandb
        except ImportError:
            return
        run_id = None
        if resume_from is not None:
            side = resume_from.parent.parent / "wandb_run_id.txt"
            if side.is_file():
                run_id = side.read_text().strip() or None
        try:
            self.wandb_run = wandb.init(project=job.wandb_project, entity=job.wandb_entity, name=job.wandb_run_name,
                                        tags=list(job.wandb_tags), id=run_id, resume="allow" if run_id else None,
                                        dir=str(self.run_dir), config=config_to_dict(job))
            (self.run_dir / "wandb_run_id.txt").write_text(self.wandb_run.id + "\n")
            nlog.set_wandb_run(self.wandb_run)
        except Exception as exc:  # wandb problems never stop training
            self.logger.warning("wandb init failed: %s", exc)

    def close(self) -> None:
        if self.wandb_run is not None:
            self.wandb_run.finish()
            nlog.set_wandb_run(None)


class TrainPipeline:
    def __init__(self, job_config: TrainJobConfig, experiment_config: ExperimentConfig) -> None:
        self.job, self.experiment = job_config, experiment_config
        self.ctx: RunContext | None = None
        self.trainer: Trainer | None = None

    @classmethod
    def from_config(cls, job_config: TrainJobConfig, experiment_config: ExperimentConfig) -> "TrainPipeline":
        return cls(job_config, experiment_config)

    def setup(self) -> Trainer:
        ctx = self.ctx = RunContext(self.job, self.experiment)
        job = self.job
        exp_dir = Path(self.experiment.output_root) / self.experiment.name
        latest, _ = find_latest_checkpoint(exp_dir, exclude_run_dir=ctx.run_dir,
                                           checkpoint_dir=job.checkpoint_dir or "checkpoints")
        path, strict, why = resolve_resume_checkpoint(
            explicit=job.resume_model_checkpoint, explicit_strict=job.resume_strict, latest_own=latest)
        ctx.init_wandb(resume_from=path if why == "auto" else None)
        dataset = build_dataset(job.train_dataset)
        loader = PinnedWindowLoader(dataset, job.train_dataloader, rank=get_rank(), world=get_world_size(),
                                    seed=0)
        model = Model.from_config(job.model)
        eval_suite = None
        if job.eval_suite is not None and job.eval_suite.evals:
            from nestor_b200.eval.suite import EvalSuite
            eval_suite = EvalSuite(job.eval_suite, device=ctx.device)
        self.trainer = Trainer(job, model, loader, device=ctx.device, run_dir=ctx.run_dir,
                               eval_suite=eval_suite, logger=ctx.logger)
        n_params = sum(p.numel() for p in model.parameters())
        ctx.logger.info("model: %s parameters (%s trainable), compute dtype %s, world %d", f"{n_params:,}",
                        f"{self.trainer.arena.numel:,}", self.trainer.compute_dtype, get_world_size())
        if path is not None:
            ctx.logger.info("[resume] %s checkpoint %s", why, path)
            self.trainer.resume(path, strict=strict,
                                allow_partial=os.environ.get("DCLM_INIT_ALLOW_PARTIAL") == "1")
        return self.trainer

    def run(self) -> None:
        trainer = self.setup()
        try:
            trainer.train()
        finally:
            assert self.ctx is not None
            self.ctx.close()


class EvalPipeline:
    def __init__(self, job_config: EvalJobConfig, experiment_config: ExperimentConfig) -> None:
        self.job, self.experiment = job_config, experiment_config

    @classmethod
    def from_config(cls, job_config: EvalJobConfig, experiment_config: ExperimentConfig) -> "EvalPipeline":
        return cls(job_config, experiment_config)

    def run(self) -> dict[str, Any]:
        from nestor_b200.eval.suite import EvalSuite
        from nestor_b200.train.checkpoint import load_checkpoint

        ctx = RunContext(self.job, self.experiment)
        model = Model.from_config(self.job.model).to(ctx.device)
        load_checkpoint(self.job.model_checkpoint_path, model, strict=False)
        results = EvalSuite(self.job.eval_suite, device=ctx.device).run(model)
        if is_main_process():
            if self.job.output_format in ("json", "both"):
                (ctx.run_dir / "eval_results.json").write_text(json.dumps(results, indent=2))
            if self.job.output_format in ("markdown", "both"):
                lines = ["| eval | metric | value |", "|---|---|---|"]
                for name, metrics in results.items():
                    for k, v in metrics.items():
                        if isinstance(v, (int, float)):
                            lines.append(f"| {name} | {k} | {v:.6g} |")
                (ctx.run_dir / "eval_results.md").write_text("\n".join(lines) + "\n")
        ctx.close()
        return results
