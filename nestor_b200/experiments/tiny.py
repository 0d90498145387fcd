"""``nestor_tiny``: a CPU-sized Nestor for plumbing checks.

Two single-layer blocks, ``d = 128``, four attention columns with top-2 routing (then a
dense ``k = G`` tail block), two heads per column, a hybrid pool of 4 public + 2 private
experts per column, the column depth read. Same recipe and ``DCLM_*`` knobs as the
pretraining cells; defaults are sized for seconds on a CPU (sequence 256, batch 2).
"""

from __future__ import annotations

import os
from pathlib import Path

from nestor_b200.configs import (
    CausalLMLossConfig, CosineAnnealingConfig, DataLoaderConfig, DclmDatasetConfig, DistributedConfig,
    ExperimentConfig, LanguageModelingHeadConfig, MuonAdamWConfig, NestorConfig, ReferenceMupConfig,
    SequenceModelConfig, TextAdapterConfig, TrainJobConfig,
)
from nestor_b200.experiments.pretrain import LR_ADAMW, LR_MUON, NESTOR_READ, REFERENCE_MUP, WEIGHT_DECAY
from nestor_b200.experiments.registry import register_experiment

TINY_VOCAB = 100_277


def tiny_backbone(dim: int = 128) -> NestorConfig:
    n = 2
    return NestorConfig(
        input_dim=dim, num_blocks=n, feature_dims=[dim] * n, causal=True, pooling_strides=[1] * n,
        block_num_layers=[1, 1], num_groups=[4, 4], num_groups_per_token=[2, 4], block_num_heads=[2, 2],
        block_head_dims=16, attention_token_dispatch=True, block_mlp_hidden_dims=[[4 * dim]] * n,
        block_mlp_activations="swiglu", router_num_experts_per_group=[1] * n, router_num_shared_experts=[1] * n,
        router_num_experts_per_group_per_token=[1] * n, router_loss_free_balancing=True,
        router_bias_update_rate=1e-3, router_score_mlp_hidden_dims=[[32]] * n,
        router_noise_mlp_hidden_dims=[[32]] * n, block_expert_pool_public_experts=[4] * n,
        block_expert_pool_public_top_k=[2] * n, block_expert_pool_private_experts=[2] * n,
        block_expert_pool_private_top_k=[2, 1], block_expert_pool_private_gate="switch", **NESTOR_READ,
    )


@register_experiment
def nestor_tiny() -> ExperimentConfig:
    block = int(os.environ.get("DCLM_BLOCK_SIZE", "256"))
    steps = int(os.environ.get("DCLM_MAX_STEPS", "4"))
    backbone = tiny_backbone()
    init_ckpt = os.environ.get("DCLM_INIT_CHECKPOINT", "").strip()     # weights-only start, as for the pretraining cells
    job = TrainJobConfig(
        name="nestor_tiny_train",
        model=SequenceModelConfig(
            adapter_config=TextAdapterConfig(tokenizer="cl100k_base", embed_dim=128, max_length=block,
                                             vocab_size=TINY_VOCAB),
            backbone_config=backbone,
            head_config=LanguageModelingHeadConfig(vocab_size=TINY_VOCAB),
            reference_mup=ReferenceMupConfig(matrix_optimizer="muon", num_layers=2, **REFERENCE_MUP)),
        train_dataset=DclmDatasetConfig(
            data_path=Path(os.environ.get("DCLM_DATA_PATH", "data/dclm/dclm_train.bin")), block_size=block),
        train_dataloader=DataLoaderConfig(batch_size=int(os.environ.get("DCLM_GLOBAL_BATCH", "2")), num_workers=0),
        optimizer=MuonAdamWConfig(lr_muon=LR_MUON, lr_adamw=LR_ADAMW, weight_decay=WEIGHT_DECAY),
        scheduler=CosineAnnealingConfig(T_max=steps, warmup_steps=int(os.environ.get("DCLM_WARMUP_STEPS", "1")),
                                        eta_min=1e-5),
        max_steps=steps, grad_accum_steps=int(os.environ.get("DCLM_GRAD_ACCUM", "1")), max_grad_norm=1.0,
        use_amp=True, loss=CausalLMLossConfig(), checkpoint_frequency=int(os.environ.get("DCLM_CKPT_FREQ", "2")),
        log_frequency=int(os.environ.get("DCLM_LOG_FREQ", "1")), distributed=DistributedConfig(enabled=True),
        wandb_project=None, seed=int(os.environ.get("DCLM_SEED", "42")),
        resume_model_checkpoint=Path(init_ckpt) if init_ckpt else None, resume_strict=not init_ckpt,
    )
    return ExperimentConfig(name="nestor_tiny", jobs=[job],
                            output_root=Path(os.environ.get("NESTOR_OUTPUT_ROOT", "./outputs")))
