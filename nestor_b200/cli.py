"""``nestor_cli``: run a registered experiment.

``nestor_cli --experiment NAME`` runs every job of the experiment in order (train jobs
through ``TrainPipeline``, eval jobs through ``EvalPipeline``); ``--list-experiments`` prints
the registry. A ``.env`` file in the working directory is loaded first (without
overriding variables already set). The process group is torn down on exit. Reference:
``nestor/cli.py:25-186``.
"""

from nestor_b200.utils import timing as _timing  # noqa: F401  (first import: stamps process start)

import argparse
import os
import sys
from pathlib import Path


def _load_dotenv(path: Path = Path(".env")) -> None:
    if not path.is_file():
        return
    for raw in path.read_text().splitlines():
        line = raw.strip()
        if not line or line.startswith("#") or "=" not in line:
            continue
        key, _, value = line.partition("=")
        key = key.removeprefix("export ").strip()
        os.environ.setdefault(key, value.strip().strip("'\""))


def _parse_args(argv: list[str] | None = None) -> argparse.Namespace:
    p = argparse.ArgumentParser(prog="nestor_cli", description="Run a registered Nestor experiment.")
    p.add_argument("--experiment", "-e", type=str, default=None, help="registered experiment name")
    p.add_argument("--list-experiments", action="store_true", help="print the registered experiments and exit")
    return p.parse_args(argv)


def main(argv: list[str] | None = None) -> int:
    _load_dotenv()
    args = _parse_args(argv)
    from nestor_b200.configs import EvalJobConfig, TrainJobConfig
    from nestor_b200.experiments import discover_experiments, get_experiment, list_experiments
    from nestor_b200.utils.distributed import cleanup_distributed

    discover_experiments()
    if args.list_experiments:
        names = list_experiments()
        print("Available experiments:" if names else "No experiments registered.")
        for n in names:
            print(f"  - {n}")
        return 0
    if not args.experiment:
        print("Error: --experiment is required. Use --list-experiments to see available options.")
        return 1
    try:
        fn = get_experiment(args.experiment)
    except KeyError as exc:
        print(f"Error: {exc}")
        return 1
    print(f"Running experiment: {args.experiment}")
    from nestor_b200.utils.flags import report_reference_flags
    from nestor_b200.utils.logging import get_logger
    report_reference_flags(get_logger("nestor_b200"))
    experiment = fn()
    experiment.name = args.experiment
    from nestor_b200.pipelines import EvalPipeline, TrainPipeline
    try:
        for i, job in enumerate(experiment.jobs):
            print(f"\n{'=' * 60}\nJob {i + 1}/{len(experiment.jobs)}: {job.name}\n{'=' * 60}\n")
            if isinstance(job, TrainJobConfig):
                TrainPipeline.from_config(job_config=job, experiment_config=experiment).run()
            elif isinstance(job, EvalJobConfig):
                EvalPipeline.from_config(job_config=job, experiment_config=experiment).run()
            else:
                print(f"Warning: unknown job type '{job.job_type}', skipping.")
        print(f"\n{'=' * 60}\nExperiment complete!\n{'=' * 60}")
    finally:
        cleanup_distributed()
    return 0


if __name__ == "__main__":
    sys.exit(main())
