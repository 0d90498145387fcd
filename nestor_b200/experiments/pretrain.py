"""The twelve pretraining cells: {dense, moe, nestor} x {100m, 200m, 500m, 1b}.

Geometry, recipe and the ``DCLM_*`` environment knobs reproduce
``nestor/experiments/pretrain.py`` of the reference (scales ``:145-150``, batch shapes
``:153-161``, column schedule ``:174-203``, job assembly ``:378-483``). One recipe
everywhere: 4096-token context, reference muP with Muon (0.01) on matrices and
AdamW (3e-4) elsewhere, weight decay 0.1, cosine to 1e-5 after 8 % warmup, clip 1.0,
seed 42.

The cells are generated from the tables below instead of being written out one by
one; ``ARMS`` maps a family name to its backbone builder.
"""

from __future__ import annotations

import dataclasses as dc
import os
from pathlib import Path
from typing import Callable

from nestor_b200.configs import (
    CausalLMLossConfig, CosineAnnealingConfig, DataLoaderConfig, DclmDatasetConfig,
    DistributedConfig, ExperimentConfig, LanguageModelingHeadConfig, MuonAdamWConfig,
    NestorConfig, ReferenceMupConfig, SequenceModelConfig, TextAdapterConfig, TrainJobConfig,
    private_expert_hidden_dim, round_to_multiple_of_8,
)
from nestor_b200.experiments.registry import register_experiment

TOKENIZER = "cl100k_base"
VOCAB_SIZE = 100_263            # cl100k ordinary tokens + end-of-text remapped to 100261
TOKEN_REMAP = {100_257: 100_261}
SERIES_BLOCK_SIZE = 4096

LR_MUON, LR_ADAMW, WEIGHT_DECAY = 0.01, 3e-4, 0.1
ROUTER_BIAS_UPDATE_RATE = 1e-3
REFERENCE_MUP = dict(width_multiplier=8.0, embedding_multiplier=12.0, residual_multiplier=0.22)


def _env(name: str, default: object) -> str:
    return os.environ.get(name, str(default))


@dc.dataclass(frozen=True)
class Scale:
    """One rung: width ``d = 40 * num_layers``, head width ``d/16``, dense MLP ``4d``, budget."""

    name: str
    hidden_size: int
    num_layers: int
    head_dim: int
    mlp_hidden: int
    max_steps: int
    warmup: int
    tokens_per_step: int

    @property
    def total_tokens(self) -> int:
        return self.max_steps * self.tokens_per_step


SCALES: dict[str, Scale] = {
    s.name: s
    for s in (
        Scale("100m", 480, 12, 30, 1920, 19_080, 1526, 262_144),
        Scale("200m", 640, 16, 40, 2560, 19_080, 1526, 524_288),
        Scale("500m", 960, 24, 60, 3840, 23_844, 1908, 1_048_576),
        Scale("1b", 1280, 32, 80, 5120, 23_842, 1907, 2_097_152),
    )
}

# (family, scale) -> (global_batch, grad_accum); product x 4096 = the rung's tokens/step.
BATCH_SHAPE: dict[tuple[str, str], tuple[int, int]] = {}
for _scale, _shapes in {"100m": (16, 4), "200m": (16, 8), "500m": (16, 16), "1b": (64, 8)}.items():
    for _family in ("dense", "moe", "nestor"):
        BATCH_SHAPE[(_family, _scale)] = _shapes
BATCH_SHAPE[("moe", "1b")] = (32, 16)

BASELINE_BLOCKS, BASELINE_HEADS, MOE_EXPERTS, BANK_TOP_K = 4, 16, 24, 3

NESTOR_COLUMNS = 8
NESTOR_TOP_K = (3, 4, 5, 6, 6, 7, 8)
NESTOR_HEADS = (5, 4, 3, 3, 3, 2, 2)
NESTOR_LAYERS = {
    "100m": (1, 1, 2, 2, 2, 3, 2),
    "200m": (2, 2, 2, 3, 3, 3, 2),
    "500m": (3, 3, 3, 4, 4, 5, 3),
    "1b": (3, 4, 4, 6, 6, 6, 4),
}
NESTOR_PUBLIC_EXPERTS, NESTOR_PUBLIC_TOP_K = 8, 2
NESTOR_PRIVATE_EXPERTS = {"100m": 8, "200m": 8, "500m": 12, "1b": 15}
NESTOR_MIN_PRIVATE_WIDTH = 160
NESTOR_READ = dict(
    block_residual_mode="attn_res_column",
    block_column_include_aggregate=True,
    block_column_gain_init=0.0,
    block_column_head_only=True,
    block_column_deviation_sources=True,
)


def moe_expert_width(scale: Scale) -> int:
    """Per-expert width of the baselines' bank: ``round8(4d / 3)``."""

    return round_to_multiple_of_8(scale.mlp_hidden / BANK_TOP_K)


def nestor_private_top_k(scale: Scale) -> tuple[int, ...]:
    """Top-2 private experts wherever they would stay at least 160 wide, else top-1."""

    return tuple(
        2 if private_expert_hidden_dim(scale.hidden_size, k, 2) >= NESTOR_MIN_PRIVATE_WIDTH else 1
        for k in NESTOR_TOP_K
    )


def _decoder(scale: Scale, *, columns, top_k, heads, layers, bank=(1, 1, None), pool=None, **read) -> NestorConfig:
    n = len(top_k)
    bank_experts, bank_top_k, bank_width = bank
    bank_width = scale.mlp_hidden if bank_width is None else bank_width
    pool_kwargs = {}
    if pool is not None:
        P, k_p, Q, k_q = pool
        pool_kwargs = dict(
            block_expert_pool_public_experts=[P] * n,
            block_expert_pool_public_top_k=[k_p] * n,
            block_expert_pool_private_experts=[Q] * n,
            block_expert_pool_private_top_k=list(k_q),
            block_expert_pool_private_gate="switch",
        )
    return NestorConfig(
        input_dim=scale.hidden_size,
        num_blocks=n,
        feature_dims=[scale.hidden_size] * n,
        causal=True,
        pooling_strides=[1] * n,
        block_num_layers=list(layers),
        num_groups=list(columns),
        num_groups_per_token=list(top_k),
        block_num_heads=list(heads),
        block_head_dims=scale.head_dim,
        attention_token_dispatch=True,
        block_mlp_hidden_dims=[[bank_width]] * n,
        block_mlp_activations="swiglu",
        router_num_experts_per_group=[bank_experts] * n,
        router_num_shared_experts=[bank_experts] * n,
        router_num_experts_per_group_per_token=[bank_top_k] * n,
        router_loss_free_balancing=True,
        router_bias_update_rate=ROUTER_BIAS_UPDATE_RATE,
        router_score_mlp_hidden_dims=[[128]] * n,
        router_noise_mlp_hidden_dims=[[128]] * n,
        **pool_kwargs,
        **read,
    )


def baseline_backbone(scale: Scale, *, experts: int) -> NestorConfig:
    """Dense attention (1 column x 16 heads), four equal blocks, Kimi depth read, expert bank."""

    assert scale.num_layers % BASELINE_BLOCKS == 0
    n = BASELINE_BLOCKS
    bank = (1, 1, scale.mlp_hidden) if experts == 1 else (experts, BANK_TOP_K, moe_expert_width(scale))
    return _decoder(
        scale, columns=(1,) * n, top_k=(1,) * n, heads=(BASELINE_HEADS,) * n,
        layers=(scale.num_layers // n,) * n, bank=bank, block_residual_mode="attn_res_kimi",
    )


def nestor_backbone(scale: Scale) -> NestorConfig:
    """Eight columns on the ``k = (3..8)`` schedule, hybrid pool, column depth read."""

    return _decoder(
        scale, columns=(NESTOR_COLUMNS,) * len(NESTOR_TOP_K), top_k=NESTOR_TOP_K, heads=NESTOR_HEADS,
        layers=NESTOR_LAYERS[scale.name],
        pool=(NESTOR_PUBLIC_EXPERTS, NESTOR_PUBLIC_TOP_K, NESTOR_PRIVATE_EXPERTS[scale.name],
              nestor_private_top_k(scale)),
        **NESTOR_READ,
    )


ARMS: dict[str, Callable[[Scale], NestorConfig]] = {
    "dense": lambda s: baseline_backbone(s, experts=1),
    "moe": lambda s: baseline_backbone(s, experts=MOE_EXPERTS),
    "nestor": nestor_backbone,
}


def build_experiment(family: str, scale_name: str) -> ExperimentConfig:
    """Assemble ``<family>_<scale>``; every smoke-vs-full difference comes from ``DCLM_*`` env."""

    scale = SCALES[scale_name]
    backbone = ARMS[family](scale)
    block_size = int(_env("DCLM_BLOCK_SIZE", SERIES_BLOCK_SIZE))
    data_path = Path(_env("DCLM_DATA_PATH", "data/dclm/dclm_train.bin"))
    cell = f"{family}_{scale.name}"
    default_gb, default_ga = BATCH_SHAPE[(family, scale.name)]
    global_batch = int(_env("DCLM_GLOBAL_BATCH", default_gb))
    grad_accum = int(_env("DCLM_GRAD_ACCUM", default_ga))
    if block_size == SERIES_BLOCK_SIZE and global_batch * grad_accum * block_size != scale.tokens_per_step:
        raise AssertionError(
            f"{cell}: {global_batch} x {grad_accum} x {block_size} != {scale.tokens_per_step:,} tokens/step"
        )
    max_steps = int(_env("DCLM_MAX_STEPS", scale.max_steps))
    warmup = int(_env("DCLM_WARMUP_STEPS", scale.warmup))
    suffix = os.environ.get("DCLM_RUN_SUFFIX", "").strip()
    run_name = f"{cell}_{suffix}" if suffix else cell
    init_ckpt = os.environ.get("DCLM_INIT_CHECKPOINT", "").strip()
    rope_base = os.environ.get("DCLM_ROPE_BASE", "").strip()
    if rope_base:
        backbone = dc.replace(backbone, block_rope_bases=float(rope_base))
    tags = [t.strip() for t in os.environ.get("WANDB_TAGS", "").split(",") if t.strip()]

    job = TrainJobConfig(
        name=f"{run_name}_train",
        model=SequenceModelConfig(
            adapter_config=TextAdapterConfig(
                tokenizer=TOKENIZER, embed_dim=scale.hidden_size, max_length=block_size, vocab_size=VOCAB_SIZE),
            backbone_config=backbone,
            head_config=LanguageModelingHeadConfig(vocab_size=VOCAB_SIZE),
            reference_mup=ReferenceMupConfig(
                matrix_optimizer="muon", num_layers=sum(backbone.block_num_layers), **REFERENCE_MUP),
        ),
        train_dataset=DclmDatasetConfig(
            data_path=data_path, block_size=block_size, tokenizer=TOKENIZER, split="train",
            token_remap=dict(TOKEN_REMAP)),
        train_dataloader=DataLoaderConfig(
            batch_size=global_batch, num_workers=int(_env("DCLM_NUM_WORKERS", 8)), drop_last=True, shuffle=True),
        optimizer=MuonAdamWConfig(
            lr_muon=float(_env("DCLM_LR_MUON", LR_MUON)), lr_adamw=float(_env("DCLM_LR_ADAMW", LR_ADAMW)),
            weight_decay=float(_env("DCLM_WEIGHT_DECAY", WEIGHT_DECAY)), betas=(0.9, 0.95)),
        scheduler=CosineAnnealingConfig(T_max=max_steps, warmup_steps=warmup, eta_min=1e-5),
        max_steps=max_steps,
        grad_accum_steps=grad_accum,
        max_grad_norm=1.0,
        use_amp=True,
        loss=CausalLMLossConfig(),
        eval_suite=None,
        eval_frequency=10_000_000,
        checkpoint_frequency=int(_env("DCLM_CKPT_FREQ", 2000)),
        log_frequency=int(_env("DCLM_LOG_FREQ", 20)),
        distributed=DistributedConfig(enabled=True),
        wandb_project=os.environ.get("WANDB_PROJECT") or "nestor",
        wandb_entity=os.environ.get("WANDB_ENTITY") or None,
        wandb_run_name=run_name,
        wandb_tags=["pretrain", family, scale.name, *tags],
        seed=int(_env("DCLM_SEED", 42)),
        resume_model_checkpoint=Path(init_ckpt) if init_ckpt else None,
        resume_strict=not init_ckpt,
    )
    tokens = global_batch * grad_accum * block_size
    print(
        f"[pretrain] {run_name}: d={scale.hidden_size} L={sum(backbone.block_num_layers)} ctx={block_size} "
        f"rope={backbone.block_rope_bases} init={init_ckpt or '-'} | {max_steps} steps x {tokens:,} tok/step = "
        f"{max_steps * tokens / 1e9:.2f}B tokens | data={data_path}"
    )
    return ExperimentConfig(
        name=run_name, jobs=[job], output_root=Path(_env("NESTOR_OUTPUT_ROOT", "./outputs")))


_DOC = {
    "dense": "Dense transformer baseline",
    "moe": "MoE control (24 experts, top-3)",
    "nestor": "Nestor (8 columns, hybrid public+private pool, column depth read)",
}


def _register_cells() -> None:
    for family in ARMS:
        for scale_name in SCALES:
            def cell(family: str = family, scale_name: str = scale_name) -> ExperimentConfig:
                return build_experiment(family, scale_name)

            cell.__name__ = cell.__qualname__ = f"{family}_{scale_name}"
            cell.__doc__ = f"{_DOC[family]} at the {scale_name} rung."
            globals()[cell.__name__] = register_experiment(cell)


_register_cells()
