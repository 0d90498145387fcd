"""Model-composition configs: adapter, head, backbone (``NestorConfig``), reference muP.

``NestorConfig`` keeps the reference's field names (``nestor/backbones/nestor.py:2031-2377``)
because experiment functions and saved ``config.json`` files are written in terms
of them. ``NestorConfig.resolve()`` expands the per-block scalars/lists into a list
of :class:`BlockSpec` records, the flat description the module tree, the kernels'
plan builders and the FLOP formulas all read.

Scope: stride-1, constant-width blocks in every residual topology of the reference (the Kimi depth read
``attn_res_kimi``, the column depth read ``attn_res_column`` with its read / export / subset variants, the plain
``projection`` stream, the between-block ``attn_res`` mixture, the within-block history attention), causal or
bidirectional, with pools, banks (shared or column-specific experts, per-layer sizes) and gated or pointwise
experts. The reference's vision-era knobs that change the token count or the width between blocks (pooling,
global tokens, per-block ``feature_dims``) are accepted at their default values only; ``resolve()`` raises on
anything else rather than silently building a different model.
"""

from __future__ import annotations

import dataclasses as dc
from typing import Any, Literal

__all__ = [
    "AdapterConfig", "TextAdapterConfig", "HeadConfig", "LanguageModelingHeadConfig",
    "BackboneConfig", "NestorConfig", "BlockSpec", "ModelConfig", "SequenceModelConfig",
    "ReferenceMupConfig", "REFERENCE_MUP_COMPONENTS",
    "round_to_multiple_of_8", "public_expert_hidden_dim", "private_expert_hidden_dim",
]

_kw = dc.dataclass(kw_only=True)


def round_to_multiple_of_8(value: float) -> int:
    """Nearest multiple of 8, never below 8 (reference: ``expert_pool_dispatch.py:25-35``)."""

    return max(8, int(round(value / 8.0)) * 8)


def public_expert_hidden_dim(dim: int, public_top_k: int, *, active_budget: float | None = None) -> int:
    """Public-pool SwiGLU width: the family's ``2d`` active budget split over ``k_p``."""

    budget = 2.0 if active_budget is None else float(active_budget)
    return round_to_multiple_of_8(budget * dim / public_top_k)


def private_expert_hidden_dim(
    dim: int, num_groups_per_token: int, private_top_k: int, *,
    with_public_pool: bool = True, active_budget: float | None = None,
) -> int:
    """Private-pool SwiGLU width: ``2d`` (``4d`` without a public pool) over ``k_a * k_q``."""

    budget = float(active_budget) if active_budget is not None else (2.0 if with_public_pool else 4.0)
    return round_to_multiple_of_8(budget * dim / (num_groups_per_token * private_top_k))


@_kw
class AdapterConfig:
    adapter_type: str = "base"


@_kw
class TextAdapterConfig(AdapterConfig):
    adapter_type: Literal["text"] = "text"
    tokenizer: str = "gpt2"
    embed_dim: int = 768
    max_length: int = 256
    vocab_size: int | None = None


@_kw
class HeadConfig:
    head_type: str = "base"


@_kw
class LanguageModelingHeadConfig(HeadConfig):
    head_type: Literal["language_modeling"] = "language_modeling"
    vocab_size: int
    hidden_dims: list[int] = dc.field(default_factory=list)
    activation: str = "gelu"


@_kw
class BackboneConfig:
    backbone_type: str = "base"


REFERENCE_MUP_COMPONENTS = (
    "architecture", "residual", "embedding", "logits", "initialization", "optimizer", "router",
)


@_kw
class ReferenceMupConfig:
    """The paper's muP parameterisation (reference: ``configs/reference_mup.py:19-94``)."""

    components: tuple[str, ...] = REFERENCE_MUP_COMPONENTS
    matrix_optimizer: str = "adamw"
    group_router_lr: str = "native"
    initializer_range: float = 0.1
    width_multiplier: float = 8.0
    embedding_multiplier: float = 12.0
    residual_multiplier: float = 0.22
    norm_eps: float = 1e-5
    num_layers: int = 40

    def __post_init__(self) -> None:
        unknown = set(self.components) - set(REFERENCE_MUP_COMPONENTS)
        if unknown:
            raise ValueError(f"Unknown reference muP components: {sorted(unknown)}")
        if self.matrix_optimizer not in ("adamw", "muon"):
            raise ValueError(f"matrix_optimizer must be 'adamw' or 'muon', got {self.matrix_optimizer!r}.")
        if self.group_router_lr not in ("native", "base"):
            raise ValueError(f"group_router_lr must be 'native' or 'base', got {self.group_router_lr!r}.")
        if self.width_multiplier <= 0 or self.num_layers <= 0:
            raise ValueError("width_multiplier and num_layers must be positive.")

    def enabled(self, component: str) -> bool:
        return component in self.components


@dc.dataclass(frozen=True)
class BlockSpec:
    """One block of the decoder, fully resolved.

    ``G`` columns of ``heads`` heads (``head_dim`` each); a token is routed to ``k``
    of them for the whole block. The MLP is either a bank of ``bank_experts`` SwiGLU
    experts of width ``bank_width`` routed top-``bank_top_k`` (``pool == False``) or the
    hybrid pool: ``P`` public experts (top-``k_p``, width ``h_pub``) plus ``Q`` private
    experts per column (top-``k_q``, width ``h_priv``).
    """

    index: int
    dim: int
    layers: int
    G: int
    k: int
    heads: int
    head_dim: int
    rope_base: float
    pool: bool
    bank_experts: int
    bank_top_k: int
    bank_width: int
    P: int
    k_p: int
    h_pub: int
    Q: int
    k_q: int
    h_priv: int
    private_gate: str
    router_hidden: int
    loss_free: bool
    bias_rate: float
    token_dispatch: bool
    dense_shared: int = 0        # always-on SwiGLU experts of the bank's width beside the routed bank (unit gate)
    layer_experts: tuple[int, ...] | None = None   # bank size per layer (None: ``bank_experts`` everywhere)
    bank_shared: int | None = None   # how many of a bank's choices are experts shared by all columns (None: all); the
                                     # other choices name one expert per column
    causal: bool = True          # False: every member of a column attends to all members of its sequence
    activation: str = "swiglu"   # bank / dense experts: 'swiglu' (gated) or a pointwise 'relu' / 'gelu' / 'silu' / 'tanh'
    columns: bool = True         # column mode: the block tracks per-column streams and exports them
    column_layers: int | None = None   # column mode: only this many trailing layers track streams (None = all)
    column_aggregate: bool = True      # column mode, k > 1: the mean of the streams is a further export
    column_deviation: bool = True      # column mode, k > 1: columns are exported / read as ``s_j - mean``
    column_head_only: bool = True      # column mode: sublayer reads see one aggregate per block; only the head read
                                       # sees the columns (False: every read sees every column)

    @property
    def inner(self) -> int:
        return self.heads * self.head_dim

    def experts_of_layer(self, layer: int) -> int:
        """Routed experts in the bank of layer ``layer`` of this block."""

        return self.bank_experts if self.layer_experts is None else self.layer_experts[layer]

    @property
    def exports(self) -> int:
        """Depth sources this block exports in column mode (k columns + the aggregate if it is exported; one for a
        merged or single-column block)."""

        return self.k + int(self.column_aggregate) if self.k > 1 and self.columns else 1

    @property
    def merged_prefix(self) -> int:
        """Leading layers of a column block that run the merged recurrence (0 unless ``column_layers`` narrows it)."""

        if not self.columns or self.column_layers is None or self.column_layers >= self.layers:
            return 0
        return self.layers - self.column_layers


def _per_block(value: Any, n: int, name: str) -> list[Any]:
    if isinstance(value, (list, tuple)):
        if len(value) != n:
            raise ValueError(f"{name} has {len(value)} entries for {n} blocks.")
        return list(value)
    return [value] * n


@_kw
class NestorConfig(BackboneConfig):
    backbone_type: Literal["nestor"] = "nestor"
    input_dim: int
    num_blocks: int
    feature_dims: list[int]
    pooling_strides: int | list[int] = 1
    pooling_keep_ratios: float | list[float] | None = None
    causal: bool = False
    block_num_layers: int | list[int] = 1
    num_groups: int | list[int] = 1
    num_groups_per_token: int | list[int] = 1
    block_num_heads: int | list[int] = 1
    block_head_dims: int | list[int] = 64
    block_rope_bases: float | list[float] = 10000.0
    block_mlp_hidden_dims: list[int] | list[list[int]] = dc.field(default_factory=lambda: [256])
    block_mlp_activations: str | list[str] = "gelu"
    router_num_experts_per_group: int | list[int] = 1
    block_layer_num_experts: list[list[int]] | None = None
    router_num_shared_experts: int | list[int] = 0
    router_num_dense_shared_experts: int | list[int] = 0
    router_num_experts_per_group_per_token: int | list[int] = 1
    router_score_mlp_hidden_dims: list[int] | list[list[int]] = dc.field(default_factory=lambda: [128])
    router_score_mlp_activations: str | list[str] = "gelu"
    router_noise_mlp_hidden_dims: list[int] | list[list[int]] = dc.field(default_factory=lambda: [128])
    router_noise_mlp_activations: str | list[str] = "gelu"
    router_loss_free_balancing: bool | list[bool] = False
    router_bias_update_rate: float | list[float] = 0.0
    attention_token_dispatch: bool | list[bool] = False
    block_expert_pool_public_experts: int | list[int] = 0
    block_expert_pool_public_top_k: int | list[int] = 1
    block_expert_pool_private_experts: int | list[int] = 0
    block_expert_pool_private_top_k: int | list[int] = 1
    block_expert_pool_private_gate: str = "renorm"
    block_expert_pool_active_budget: float | None = None
    block_expert_pool_public_budget: float | None = None
    mlp_auto_dense_ratio: float | None = None
    attention_auto_head_split: bool = False
    residual_mode: str = "convex"
    block_residual_mode: str = "projection"
    block_attn_res_include_embedding: bool = True
    block_column_include_aggregate: bool = False
    block_column_gain_init: float = 1.0
    block_column_mass_lambda: float | None = None
    block_column_head_only: bool = False
    block_column_head_query_per_source: bool = False
    block_column_deviation_sources: bool = False
    block_column_blocks: list[int] | None = None
    block_column_trailing_layers: int | None = None
    drop_path_rate: float = 0.0
    num_global_tokens: int = 0
    pooling_mode: str = "mean"

    # ------------------------------------------------------------------ resolution
    def resolve(self) -> list[BlockSpec]:
        """Validate and expand into one :class:`BlockSpec` per block."""

        n = self.num_blocks
        if n < 1:
            raise ValueError("num_blocks must be positive.")
        if len(self.feature_dims) != n:
            raise ValueError("feature_dims must have one entry per block.")
        if any(d != self.input_dim for d in self.feature_dims):
            raise ValueError("Only constant-width decoders are supported (feature_dims == input_dim).")
        if any(s != 1 for s in _per_block(self.pooling_strides, n, "pooling_strides")):
            raise ValueError("Token pooling between blocks is not supported (pooling_strides must be 1).")
        keep = [] if self.pooling_keep_ratios is None else _per_block(self.pooling_keep_ratios, n, "pooling_keep_ratios")
        if any(r not in (None, 1.0) for r in keep) or self.num_global_tokens:
            raise ValueError("pooling_keep_ratios (other than 1.0) / num_global_tokens are not supported: the token "
                             "count is constant through the model.")
        if not 0.0 <= self.drop_path_rate < 1.0:
            raise ValueError("drop_path_rate must be in [0, 1).")
        if self.block_residual_mode not in ("attn_res_kimi", "attn_res_column", "projection", "attn_res"):
            raise ValueError(
                "block_residual_mode must be 'projection', 'attn_res', 'attn_res_kimi' or 'attn_res_column', got "
                f"{self.block_residual_mode!r}."
            )
        if self.residual_mode not in ("convex", "attn_res"):
            raise ValueError("residual_mode must be 'convex' or 'attn_res' ('attn_res_xblock' pools over all tokens: "
                             "non-causal models only).")
        if self.residual_mode == "attn_res" and self.block_residual_mode in ("attn_res_kimi", "attn_res_column"):
            raise ValueError(f"block_residual_mode={self.block_residual_mode!r} replaces the within-block stream by "
                             "its own recurrence: it requires residual_mode='convex'.")
        if self.block_residual_mode == "attn_res_column":
            # the narrow sublayer reads are made of the aggregates, and deviations are relative to them
            if self.block_column_head_only and not self.block_column_include_aggregate:
                raise ValueError("block_column_head_only requires block_column_include_aggregate=True.")
            if self.block_column_deviation_sources and not self.block_column_include_aggregate:
                raise ValueError("block_column_deviation_sources requires block_column_include_aggregate=True.")
            if all(v <= 1 for v in _per_block(self.num_groups_per_token, n, "num_groups_per_token")):
                raise ValueError("attn_res_column needs a block with num_groups_per_token > 1; with one column per "
                                 "block everywhere it is 'attn_res_kimi', set that mode instead.")
        else:
            for name in ("block_column_head_query_per_source", "block_column_blocks", "block_column_trailing_layers",
                         "block_column_head_only", "block_column_include_aggregate", "block_column_deviation_sources"):
                if getattr(self, name) not in (None, False):
                    raise ValueError(f"{name} configures column-mode blocks: it needs block_residual_mode='attn_res_column'.")
            if self.block_column_gain_init != 1.0:
                raise ValueError("block_column_gain_init scales column sources: it needs block_residual_mode='attn_res_column'.")
        if self.block_column_gain_init < 0.0:
            raise ValueError("block_column_gain_init must be non-negative.")
        if self.block_column_mass_lambda is not None:
            # one unit of init mass per multi-column block: 1 - lambda on its aggregate, lambda / k on each column
            if not 0.0 <= self.block_column_mass_lambda <= 1.0:
                raise ValueError("block_column_mass_lambda must lie in [0, 1].")
            if not self.block_column_include_aggregate:
                raise ValueError("block_column_mass_lambda needs block_column_include_aggregate=True.")
            if self.block_column_gain_init != 1.0:
                raise ValueError("block_column_mass_lambda and a non-default block_column_gain_init both set the column gains; set one.")
        if self.block_column_trailing_layers is not None and self.block_column_trailing_layers < 1:
            raise ValueError("block_column_trailing_layers must be at least 1 (drop the block from block_column_blocks instead).")
        if self.block_column_blocks is not None:
            if not self.block_column_blocks:
                raise ValueError("block_column_blocks is empty: that is plain attn_res_kimi, set that mode instead.")
            if any(not 0 <= b < n for b in self.block_column_blocks):
                raise ValueError(f"block_column_blocks {self.block_column_blocks} has an index outside [0, {n}).")
        if self.mlp_auto_dense_ratio is not None and self.mlp_auto_dense_ratio <= 0:
            raise ValueError("mlp_auto_dense_ratio must be positive.")
        schedule = self.block_layer_num_experts
        if schedule is not None:
            # depth-varying bank sizes: one count per layer of every block, same top-k and width everywhere
            # (reference nestor/backbones/nestor.py:2131-2141, 2785-2812)
            if len(schedule) != n:
                raise ValueError("block_layer_num_experts must have one entry per block.")
            schedule = [[int(e) for e in row] for row in schedule]
            if any(e < 1 for row in schedule for e in row):
                raise ValueError("block_layer_num_experts entries must be >= 1.")
        dense_shared = _per_block(self.router_num_dense_shared_experts, n, "router_num_dense_shared_experts")
        if any(int(v) < 0 for v in dense_shared):
            raise ValueError("router_num_dense_shared_experts must be >= 0.")
        acts = _per_block(self.block_mlp_activations, n, "block_mlp_activations")
        if any(a not in ("swiglu", "relu", "gelu", "silu", "tanh") for a in acts):
            raise ValueError("block_mlp_activations must be 'swiglu' or one of 'relu', 'gelu', 'silu', 'tanh'.")

        layers = _per_block(self.block_num_layers, n, "block_num_layers")
        G = _per_block(self.num_groups, n, "num_groups")
        k = _per_block(self.num_groups_per_token, n, "num_groups_per_token")
        heads = _per_block(self.block_num_heads, n, "block_num_heads")
        hd = _per_block(self.block_head_dims, n, "block_head_dims")
        rope = _per_block(self.block_rope_bases, n, "block_rope_bases")
        if self.attention_auto_head_split:
            # a block's full head budget d / head_dim split over a token's k columns, so the active attention
            # compute matches a dense block at any k (reference nestor/backbones/nestor.py:2609-2622)
            heads = [max(1, round((self.feature_dims[i] // hd[i]) / k[i])) for i in range(n)]
        hid = self.block_mlp_hidden_dims
        hid = [list(h) for h in hid] if hid and isinstance(hid[0], (list, tuple)) else [list(hid)] * n
        epg = _per_block(self.router_num_experts_per_group, n, "router_num_experts_per_group")
        if schedule is not None:
            for i, row in enumerate(schedule):
                if len(row) != layers[i]:
                    raise ValueError(f"block_layer_num_experts[{i}] must have block_num_layers ({layers[i]}) entries, "
                                     f"got {len(row)}.")
            epg = [max(row) for row in schedule]
        shared = _per_block(self.router_num_shared_experts, n, "router_num_shared_experts")
        etop = _per_block(self.router_num_experts_per_group_per_token, n, "router_num_experts_per_group_per_token")
        if self.mlp_auto_dense_ratio is not None:
            # fine-grained experts: width = ratio * d / top_k, so the active expert FLOPs equal a dense (ratio x)
            # feed-forward at any top_k (reference nestor/backbones/nestor.py:2672-2690)
            hid = [[max(1, round(self.mlp_auto_dense_ratio * self.feature_dims[i] / etop[i]))] for i in range(n)]
        sh = self.router_score_mlp_hidden_dims
        sh = [list(h) for h in sh] if sh and isinstance(sh[0], (list, tuple)) else [list(sh)] * n
        nh = self.router_noise_mlp_hidden_dims
        nh = [list(h) for h in nh] if nh and isinstance(nh[0], (list, tuple)) else [list(nh)] * n
        lf = _per_block(self.router_loss_free_balancing, n, "router_loss_free_balancing")
        br = _per_block(self.router_bias_update_rate, n, "router_bias_update_rate")
        td = _per_block(self.attention_token_dispatch, n, "attention_token_dispatch")
        P = _per_block(self.block_expert_pool_public_experts, n, "block_expert_pool_public_experts")
        kp = _per_block(self.block_expert_pool_public_top_k, n, "block_expert_pool_public_top_k")
        Q = _per_block(self.block_expert_pool_private_experts, n, "block_expert_pool_private_experts")
        kq = _per_block(self.block_expert_pool_private_top_k, n, "block_expert_pool_private_top_k")
        if self.block_expert_pool_private_gate not in ("renorm", "switch"):
            raise ValueError("block_expert_pool_private_gate must be 'renorm' or 'switch'.")

        specs: list[BlockSpec] = []
        for i in range(n):
            if not 1 <= k[i] <= G[i]:
                raise ValueError(f"block {i}: num_groups_per_token must be in [1, num_groups].")
            if hd[i] % 2:
                raise ValueError(f"block {i}: RoPE needs an even head_dim.")
            if len(hid[i]) != 1:
                raise ValueError(f"block {i}: expert MLPs take exactly one hidden width.")
            if len(sh[i]) != 1 or len(nh[i]) != 1 or sh[i] != nh[i]:
                raise ValueError(f"block {i}: group-router score/noise MLPs need one equal hidden width.")
            pool = Q[i] > 0
            if pool:
                if P[i] < 0:
                    raise ValueError(f"block {i}: block_expert_pool_public_experts must be >= 0.")
                if epg[i] != 1 or shared[i] != 1 or int(dense_shared[i]) != 0:
                    raise ValueError(f"block {i}: the hybrid pool replaces the bank (bank experts must be 1, no dense shared experts).")
                # P == 0 is the private-only pool: no public experts, no public router, no path gate
                if not ((P[i] == 0 or 1 <= kp[i] <= P[i]) and 1 <= kq[i] <= Q[i]):
                    raise ValueError(f"block {i}: pool top-k out of range.")
            else:
                fewest = epg[i] if schedule is None else min(schedule[i])
                if G[i] > 1 and fewest == 1 and shared[i] == 0:
                    # (one unstacked dense expert per column: the stacked bank layout needs at least two choices)
                    raise ValueError(f"block {i}: column-specific experts need banks of at least two choices "
                                     "(router_num_experts_per_group > 1 in every layer).")
                if not 0 <= shared[i] <= fewest:
                    raise ValueError(f"block {i}: router_num_shared_experts must be in [0, fewest experts of a layer].")
                if not 1 <= etop[i] <= fewest:
                    raise ValueError(f"block {i}: bank top-k out of range.")
            keeps = self.column_mode and (self.block_column_blocks is None or i in self.block_column_blocks)
            specs.append(BlockSpec(
                index=i, dim=self.input_dim, layers=layers[i], G=G[i], k=k[i], heads=heads[i],
                head_dim=hd[i], rope_base=float(rope[i]), pool=pool,
                bank_experts=epg[i], bank_top_k=etop[i], bank_width=hid[i][0],
                P=P[i] if pool else 0, k_p=kp[i] if pool and P[i] > 0 else 0,
                h_pub=public_expert_hidden_dim(self.input_dim, kp[i], active_budget=self.block_expert_pool_public_budget)
                if pool and P[i] > 0 else 0,
                Q=Q[i] if pool else 0, k_q=kq[i] if pool else 0,
                # a private-only pool spends the whole 4d active width on the private experts
                h_priv=private_expert_hidden_dim(self.input_dim, k[i], kq[i], with_public_pool=P[i] > 0,
                                                 active_budget=self.block_expert_pool_active_budget) if pool else 0,
                private_gate=self.block_expert_pool_private_gate,
                router_hidden=sh[i][0], loss_free=bool(lf[i]), bias_rate=float(br[i]), token_dispatch=bool(td[i]),
                dense_shared=int(dense_shared[i]),
                layer_experts=None if pool or schedule is None else tuple(schedule[i]),
                bank_shared=None if pool else int(shared[i]),
                causal=bool(self.causal),
                activation="swiglu" if pool else acts[i],      # pool experts are always SwiGLU
                columns=keeps, column_layers=self.block_column_trailing_layers if keeps else None,
                column_aggregate=self.block_column_include_aggregate and k[i] > 1,
                column_deviation=self.block_column_deviation_sources and k[i] > 1,
                column_head_only=self.block_column_head_only,
            ))
        return specs

    @property
    def output_dim(self) -> int:
        return self.feature_dims[-1]

    @property
    def column_mode(self) -> bool:
        return self.block_residual_mode == "attn_res_column"

    @property
    def history_attention(self) -> bool:
        """``residual_mode='attn_res'``: inside a block every sublayer reads a softmax mixture of the block input and
        all earlier sublayer updates instead of a residual stream."""

        return self.residual_mode == "attn_res"

    @property
    def depth_reads(self) -> bool:
        """Whether sublayers read a softmax-over-depth mixture (the two ``attn_res_*`` modes) or the plain residual
        stream (``projection``: ``x + m * update`` under the reference muP, the convex rule otherwise)."""

        return self.block_residual_mode not in ("projection", "attn_res")

    def max_depth_sources(self) -> int:
        """Slots of the widest depth read: the embedding plus every block's exports."""

        specs = self.resolve()
        if self.column_mode:
            return 1 + sum(s.exports for s in specs)
        return 1 + len(specs)

    def to_dict(self) -> dict[str, Any]:
        """Validated plain-dict form (used for ``config.json``)."""

        self.resolve()
        return dc.asdict(self)


@_kw
class ModelConfig:
    model_type: str = "base"


@_kw
class SequenceModelConfig(ModelConfig):
    model_type: Literal["sequence"] = "sequence"
    adapter_config: AdapterConfig
    backbone_config: BackboneConfig
    head_config: HeadConfig
    reference_mup: ReferenceMupConfig | None = None
