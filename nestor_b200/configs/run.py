"""Run-level configs: data, distribution, losses, optimizers, schedules, jobs.

Parity targets (field names and defaults): ``nestor/configs/data.py``,
``distributed.py``, ``losses.py``, ``optim.py``, ``sched.py``, ``evals.py``,
``jobs.py``, ``experiment.py`` of the reference.
"""

from __future__ import annotations

import dataclasses as dc
from pathlib import Path
from typing import Any, Literal

__all__ = [
    "DatasetConfig", "DclmDatasetConfig", "DataLoaderConfig", "DistributedConfig",
    "LossConfig", "CausalLMLossConfig", "RouterBalanceLossConfig",
    "ReferenceMoEAuxLossConfig", "CompositeLossConfig",
    "OptimizerConfig", "AdamConfig", "AdamWConfig", "MuonAdamWConfig", "SGDConfig",
    "SchedulerConfig", "CosineAnnealingConfig", "WSDConfig", "PowerLawConfig", "StepLRConfig",
    "EvalConfig", "LanguageModelingEvalConfig", "EvalSuiteConfig",
    "JobConfig", "TrainJobConfig", "EvalJobConfig", "ExperimentConfig",
    "config_to_dict",
]

_kw = dc.dataclass(kw_only=True)


# ----------------------------------------------------------------------------- data
@_kw
class DatasetConfig:
    dataset_type: str = "base"
    split: Literal["train", "val", "test"] = "train"


@_kw
class DclmDatasetConfig(DatasetConfig):
    """Flat token ``.bin`` served as non-overlapping ``block_size`` windows."""

    dataset_type: Literal["dclm"] = "dclm"
    data_path: Path = dc.field(default_factory=lambda: Path("./data/dclm/dclm.bin"))
    token_dtype: Literal["uint16", "uint32"] = "uint32"
    block_size: int = 4096
    tokenizer: str = "cl100k_base"
    token_remap: dict[int, int] = dc.field(default_factory=dict)


@_kw
class DataLoaderConfig:
    batch_size: int = 32
    num_workers: int = 4
    pin_memory: bool = True
    drop_last: bool = True
    shuffle: bool = True
    prefetch_factor: int | None = 2
    persistent_workers: bool = False


# ---------------------------------------------------------------------- distribution
@_kw
class DistributedConfig:
    """Process-group settings. ``fsdp2_*`` knobs steer the sharded-parameter mode."""

    enabled: bool = False
    backend: Literal["nccl", "gloo"] = "nccl"
    init_method: str = "env://"
    world_size: int | None = None
    rank: int | None = None
    local_rank: int | None = None
    fsdp2_reshard_after_forward: bool | int | None = None
    fsdp2_param_dtype: Literal["float32", "float16", "bfloat16"] | None = None
    fsdp2_reduce_dtype: Literal["float32", "float16", "bfloat16"] | None = None
    fsdp2_output_dtype: Literal["float32", "float16", "bfloat16"] | None = None
    fsdp2_cpu_offload: bool = False


# ---------------------------------------------------------------------------- losses
@_kw
class LossConfig:
    loss_type: str = "base"


@_kw
class CausalLMLossConfig(LossConfig):
    loss_type: Literal["causal_lm"] = "causal_lm"
    label_smoothing: float = 0.0


@_kw
class RouterBalanceLossConfig(LossConfig):
    loss_type: Literal["router_balance"] = "router_balance"
    balance_weight: float = 0.01
    diversity_weight: float = 0.01


@_kw
class ReferenceMoEAuxLossConfig(LossConfig):
    loss_type: Literal["reference_moe_aux"] = "reference_moe_aux"
    coefficient: float = 0.01
    z_loss_weight: float = 0.1


@_kw
class CompositeLossConfig(LossConfig):
    loss_type: Literal["composite"] = "composite"
    losses: list[LossConfig] = dc.field(default_factory=list)
    weights: list[float] = dc.field(default_factory=list)


# ------------------------------------------------------------------------ optimizers
@_kw
class OptimizerConfig:
    optimizer_type: str = "base"
    lr: float = 1e-4
    weight_decay: float = 0.0


@_kw
class AdamConfig(OptimizerConfig):
    optimizer_type: Literal["adam"] = "adam"
    betas: tuple[float, float] = (0.9, 0.999)
    eps: float = 1e-8


@_kw
class AdamWConfig(OptimizerConfig):
    optimizer_type: Literal["adamw"] = "adamw"
    weight_decay: float = 0.01
    betas: tuple[float, float] = (0.9, 0.999)
    eps: float = 1e-8


@_kw
class MuonAdamWConfig(OptimizerConfig):
    """Muon on matrix-tagged parameters, AdamW on the rest."""

    optimizer_type: Literal["muon_adamw"] = "muon_adamw"
    lr: float = 1e-3
    lr_muon: float = 0.02
    lr_adamw: float = 1e-3
    weight_decay: float = 0.01
    betas: tuple[float, float] = (0.9, 0.95)
    eps: float = 1e-8
    muon_momentum: float = 0.95
    muon_nesterov: bool = True
    muon_ns_steps: int = 5


@_kw
class SGDConfig(OptimizerConfig):
    optimizer_type: Literal["sgd"] = "sgd"
    lr: float = 0.1
    weight_decay: float = 1e-4
    momentum: float = 0.9
    nesterov: bool = True


# ------------------------------------------------------------------------- schedules
@_kw
class SchedulerConfig:
    scheduler_type: str = "base"


@_kw
class CosineAnnealingConfig(SchedulerConfig):
    scheduler_type: Literal["cosine"] = "cosine"
    T_max: int = 100000
    eta_min: float = 1e-6
    warmup_steps: int = 1000


@_kw
class WSDConfig(SchedulerConfig):
    scheduler_type: Literal["wsd"] = "wsd"
    total_steps: int = 100000
    warmup_steps: int = 2000
    decay_steps: int = 20000
    eta_min: float = 1e-5
    decay_shape: Literal["one_minus_sqrt", "linear", "cosine"] = "one_minus_sqrt"


@_kw
class PowerLawConfig(SchedulerConfig):
    scheduler_type: Literal["power"] = "power"
    warmup_steps: int = 2000
    base_lr: float = 0.01
    a: float = 4096.0
    b: float = -0.566
    c: float = 4_194_304.0


@_kw
class StepLRConfig(SchedulerConfig):
    scheduler_type: Literal["step"] = "step"
    step_size: int = 30
    gamma: float = 0.1
    warmup_steps: int = 0


# ----------------------------------------------------------------------------- evals
@_kw
class EvalConfig:
    eval_type: str = "base"
    name: str = "eval"
    dataset_config: DatasetConfig = dc.field(default_factory=DatasetConfig)
    dataloader_config: DataLoaderConfig = dc.field(default_factory=DataLoaderConfig)


@_kw
class LanguageModelingEvalConfig(EvalConfig):
    eval_type: Literal["language_modeling"] = "language_modeling"
    name: str = "language_modeling"


@_kw
class EvalSuiteConfig:
    evals: list[EvalConfig] = dc.field(default_factory=list)


# ------------------------------------------------------------------------------ jobs
@_kw
class JobConfig:
    job_type: str = "base"
    name: str = "job"
    seed: int | None = None


@_kw
class TrainJobConfig(JobConfig):
    """One training job: model, data, optimizer, schedule, loop knobs, logging."""

    job_type: Literal["train"] = "train"
    name: str = "train"
    model: Any
    train_dataset: DatasetConfig = dc.field(default_factory=DatasetConfig)
    train_dataloader: DataLoaderConfig = dc.field(default_factory=DataLoaderConfig)
    optimizer: OptimizerConfig = dc.field(default_factory=OptimizerConfig)
    scheduler: SchedulerConfig | None = None
    max_steps: int = 100000
    grad_accum_steps: int = 1
    max_grad_norm: float | None = 1.0
    use_amp: bool = False
    ema_decay: float | None = None
    loss: LossConfig = dc.field(default_factory=LossConfig)
    eval_suite: EvalSuiteConfig | None = None
    eval_frequency: int = 1000
    checkpoint_dir: Path | None = Path("checkpoints")
    checkpoint_frequency: int = 5000
    log_frequency: int = 100
    distributed: DistributedConfig = dc.field(default_factory=DistributedConfig)
    wandb_project: str | None = None
    wandb_entity: str | None = None
    wandb_run_name: str | None = None
    wandb_tags: list[str] = dc.field(default_factory=list)
    resume_model_checkpoint: Path | None = None
    resume_strict: bool = True
    eval_submit_scripts: list[tuple[Path, int]] | None = None
    seed: int = 42


@_kw
class EvalJobConfig(JobConfig):
    job_type: Literal["eval"] = "eval"
    name: str = "eval"
    model: Any
    model_checkpoint_path: Path
    eval_suite: EvalSuiteConfig = dc.field(default_factory=EvalSuiteConfig)
    distributed: DistributedConfig = dc.field(default_factory=DistributedConfig)
    output_format: Literal["json", "markdown", "both"] = "both"
    seed: int = 42


@_kw
class ExperimentConfig:
    name: str = "experiment"
    jobs: list[JobConfig] = dc.field(default_factory=list)
    output_root: Path = dc.field(default_factory=lambda: Path("./outputs"))
    save_source_snapshot: bool = True


def config_to_dict(obj: Any) -> Any:
    """Recursively turn dataclasses / paths / tuples into JSON-serialisable values.

    Used for the per-run ``config.json`` (reference: ``nestor/pipelines/base.py:248-269``).
    """

    if dc.is_dataclass(obj) and not isinstance(obj, type):
        out = {"__class__": type(obj).__name__}
        for f in dc.fields(obj):
            out[f.name] = config_to_dict(getattr(obj, f.name))
        return out
    if isinstance(obj, Path):
        return str(obj)
    if isinstance(obj, dict):
        return {str(k): config_to_dict(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return [config_to_dict(v) for v in obj]
    if isinstance(obj, (str, int, float, bool)) or obj is None:
        return obj
    return repr(obj)
