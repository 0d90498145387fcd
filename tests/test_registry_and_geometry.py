"""Registry, geometry, parameter counts and checkpoint key schema of the registered cells.

Mirrors the pins of the reference's ``tests/test_pretrain_arms.py`` (parameter counts ``:69-73``,
private top-k ``:74-79``, FLOP ratios ``:80``) and checks the ``state_dict`` key / shape / tag schema
against fixtures captured from the reference implementation on the meta device.
"""

import json
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent

import pytest
import torch

from nestor_b200.configs import NestorConfig
from nestor_b200.continual.flops import flop_ratio
from nestor_b200.experiments import discover_experiments, get_experiment, list_experiments, register_experiment
from nestor_b200.experiments import pretrain as P
from nestor_b200.models import Model
from nestor_b200.models.tags import get_tag

FIX = Path(__file__).parent / "fixtures"
PARAMS = {
    "nestor": {"100m": 377_505_845, "200m": 761_788_781, "500m": 2_442_638_813, "1b": 5_532_512_845},
    "moe": {"100m": 373_387_389, "200m": 786_607_269, "500m": 2_405_976_309, "1b": 5_494_150_469},
    "dense": {"100m": 141_011_709, "200m": 233_903_269, "500m": 547_500_789, "1b": 1_097_053_509},
}


def _build(name):
    discover_experiments()
    with torch.device("meta"):
        return Model.from_config(get_experiment(name)().jobs[0].model)


def test_twelve_cells_registered():
    discover_experiments()
    names = list_experiments()
    for fam in ("dense", "moe", "nestor"):
        for scale in ("100m", "200m", "500m", "1b"):
            assert f"{fam}_{scale}" in names
    with pytest.raises(KeyError):
        get_experiment("nope")
    with pytest.raises(ValueError):
        register_experiment(get_experiment("nestor_200m"))


@pytest.mark.parametrize("family", ["nestor", "moe", "dense"])
@pytest.mark.parametrize("scale", ["100m", "200m", "500m", "1b"])
def test_parameter_counts(family, scale):
    model = _build(f"{family}_{scale}")
    assert sum(p.numel() for p in model.parameters()) == PARAMS[family][scale]


def test_private_top_k_and_widths():
    assert P.nestor_private_top_k(P.SCALES["200m"]) == (2, 2, 1, 1, 1, 1, 1)
    assert P.nestor_private_top_k(P.SCALES["1b"]) == (2,) * 7
    specs = P.nestor_backbone(P.SCALES["200m"]).resolve()
    assert [s.h_priv for s in specs] == [216, 160, 256, 216, 216, 184, 160]
    assert all(s.h_pub == 640 for s in specs)
    assert P.moe_expert_width(P.SCALES["200m"]) == 856
    assert P.nestor_backbone(P.SCALES["200m"]).max_depth_sources() == 47
    assert P.baseline_backbone(P.SCALES["200m"], experts=1).max_depth_sources() == 5


def test_flop_ratios():
    got = [round(flop_ratio(f"nestor_{s}", f"dense_{s}", seq_len=4096), 3) for s in ("100m", "200m", "500m", "1b")]
    assert got == [0.986, 0.981, 0.979, 0.989]
    assert abs(flop_ratio("nestor_200m", "dense_200m", seq_len=65536) - 0.8) < 0.02


@pytest.mark.parametrize("family", ["nestor", "moe", "dense"])
def test_state_dict_schema_matches_reference(family):
    schema = json.loads((FIX / f"state_schema_{family}_200m.json").read_text())
    model = _build(f"{family}_200m")
    params = dict(model.named_parameters())
    state = model.state_dict()
    assert [k for k, *_ in schema] == list(state)
    for key, shape, is_buffer, requires_grad, tag in schema:
        assert list(state[key].shape) == shape, key
        if is_buffer:
            assert key not in params
            continue
        p = params[key]
        assert bool(requires_grad) == p.requires_grad, key
        if not p.requires_grad:
            continue
        t = get_tag(p)
        assert t is not None, key
        assert t.optimizer == tag[0], key
        assert t.lr_mul == pytest.approx(tag[1], rel=1e-9), key
        assert t.muon_scale == pytest.approx(tag[2], rel=1e-9), key
        assert t.weight_decay == tag[3], key


def test_tokens_per_step_is_pinned(monkeypatch):
    monkeypatch.setenv("DCLM_GLOBAL_BATCH", "5")
    with pytest.raises(AssertionError):
        P.build_experiment("nestor", "200m")
    monkeypatch.setenv("DCLM_GLOBAL_BATCH", "32")
    monkeypatch.setenv("DCLM_GRAD_ACCUM", "4")
    job = P.build_experiment("nestor", "200m").jobs[0]
    assert job.train_dataloader.batch_size == 32 and job.grad_accum_steps == 4


def test_config_validation():
    base = dict(input_dim=64, num_blocks=1, feature_dims=[64], causal=True, block_mlp_activations="swiglu",
                block_mlp_hidden_dims=[256], block_residual_mode="attn_res_kimi", router_num_shared_experts=1)
    NestorConfig(**base).resolve()
    assert NestorConfig(**{**base, "causal": False}).resolve()[0].causal is False     # bidirectional encoders are a mode
    with pytest.raises(ValueError):
        NestorConfig(**{**base, "pooling_strides": 2}).resolve()
    with pytest.raises(ValueError):
        NestorConfig(**{**base, "causal": False, "num_global_tokens": 4}).resolve()
    with pytest.raises(ValueError):
        NestorConfig(**{**base, "block_residual_mode": "no_such_mode"}).resolve()
    NestorConfig(**{**base, "block_residual_mode": "projection"}).resolve()      # plain residual blocks are a supported mode
    with pytest.raises(ValueError):
        NestorConfig(**{**base, "num_groups": 2, "num_groups_per_token": 3}).resolve()


def test_part_registries_dispatch_on_config_type():
    import dataclasses as dc
    import pytest
    from nestor_b200.configs.model import LanguageModelingHeadConfig, NestorConfig, SequenceModelConfig, TextAdapterConfig
    from nestor_b200.models import Backbone, Nestor, SequenceModel, TextAdapter
    from nestor_b200.models.registry import ADAPTERS, BACKBONES, HEADS, MODELS, Registry
    assert MODELS.registered()[SequenceModelConfig] is SequenceModel and ADAPTERS.registered()[TextAdapterConfig] is TextAdapter
    assert NestorConfig in BACKBONES.registered() and LanguageModelingHeadConfig in HEADS.registered()
    assert issubclass(Nestor, Backbone)

    @dc.dataclass
    class Special(TextAdapterConfig):       # a subclassed config builds its parent's part
        pass

    a = ADAPTERS.build(Special(vocab_size=50, embed_dim=8), None)
    assert isinstance(a, TextAdapter)
    r = Registry("widget")
    with pytest.raises(TypeError, match="no widget registered"):
        r.build(object())
    r.register(int)(lambda c: c + 1)
    assert r.build(True) == 2                # bool -> int through the MRO
    with pytest.raises(ValueError, match="already registered"):
        r.register(int)(lambda c: c)


@pytest.mark.parametrize("family", ["nestor", "moe", "dense"])
def test_analytic_flops_agree_with_flop_counter(family, tiny_scale):
    """The analytic per-token FLOP formula against ``FlopCounterMode`` on the PyTorch statement of the model."""

    import torch
    from nestor_b200.models import Model
    from nestor_b200.train.flops import calibrate_flops, grouped_mm_flops, register_extra_flop_formulas
    torch.manual_seed(0)
    m = Model.from_config(tiny_scale.build_experiment(family, "tiny").jobs[0].model)
    cal = calibrate_flops(m, seq_len=64, batch=2)
    assert cal["counted"] > 0 and abs(cal["ratio"] - 1.0) < 0.06, cal
    assert grouped_mm_flops(10, 4, 6) == 480
    register_extra_flop_formulas(); register_extra_flop_formulas()      # idempotent


def test_auto_head_split_and_dense_ratio_follow_the_reference(tiny_scale, monkeypatch):
    """``attention_auto_head_split`` and ``mlp_auto_dense_ratio`` derive the same per-block head counts and expert
    widths as the reference's config expansion (reference nestor/backbones/nestor.py:2609-2690)."""

    import dataclasses as dc
    ref_root = ROOT / "baseline" / "_ref"
    if not (ref_root / "nestor").is_dir():
        pytest.skip("reference package not installed under baseline/_ref")
    monkeypatch.syspath_prepend(str(ref_root))
    try:
        from nestor.experiments import pretrain as RP
    except Exception as exc:
        pytest.skip(f"reference import failed: {exc}")
    P = tiny_scale
    monkeypatch.setitem(RP.SCALES, "tiny", RP.Scale("tiny", 128, 4, 8, 512, 10, 2, 1024))
    monkeypatch.setitem(RP.NESTOR_LAYERS, "tiny", (2, 1, 1, 1, 1, 1, 2))
    monkeypatch.setitem(RP.NESTOR_PRIVATE_EXPERTS, "tiny", 3)
    monkeypatch.setattr(RP, "NESTOR_MIN_PRIVATE_WIDTH", 24)
    monkeypatch.setattr(RP, "BLOCK_SIZE", 64)
    for fam in ("dense", "moe", "nestor"):
        monkeypatch.setitem(RP.BATCH_SHAPE, (fam, "tiny"), (2, 1))
    changes = dict(attention_auto_head_split=True, mlp_auto_dense_ratio=2.5)
    resolved = {}
    for fam, ref_build in (("nestor", RP._nestor), ("moe", RP._moe)):
        rcfg = ref_build("tiny").jobs[0].model.backbone_config
        ref_blocks = dc.replace(rcfg, **changes).to_dict()["block_configs"]
        ours = dc.replace(P.build_experiment(fam, "tiny").jobs[0].model.backbone_config, **changes).resolve()
        assert len(ours) == len(ref_blocks)
        for s, r in zip(ours, ref_blocks):
            assert s.heads == r["block_num_heads"]
            assert [s.bank_width] == list(r["block_mlp_hidden_dims"])
        resolved[fam] = ours
    # the derived values replace the configured ones
    base = P.build_experiment("nestor", "tiny").jobs[0].model.backbone_config
    odd = dc.replace(base, block_num_heads=1, block_mlp_hidden_dims=[8], **changes).resolve()
    assert [s.heads for s in odd] == [s.heads for s in resolved["nestor"]]
    assert [s.bank_width for s in odd] == [s.bank_width for s in resolved["nestor"]]


_COLUMN = dict(input_dim=64, num_blocks=2, feature_dims=[64, 64], causal=True, block_mlp_activations="swiglu",
               block_mlp_hidden_dims=[256], block_residual_mode="attn_res_column", router_num_shared_experts=1,
               num_groups=4, num_groups_per_token=[2, 1], block_num_layers=[2, 1],
               block_column_include_aggregate=True, block_column_head_only=True, block_column_deviation_sources=True)


@pytest.mark.parametrize("change,message", [
    (dict(block_column_mass_lambda=1.5), r"\[0, 1\]"),
    (dict(block_column_mass_lambda=0.5, block_column_gain_init=0.0), "set one"),
    (dict(block_column_mass_lambda=0.5, block_column_include_aggregate=False, block_column_head_only=False,
          block_column_deviation_sources=False), "include_aggregate"),
    (dict(block_column_include_aggregate=False), "include_aggregate"),                      # head-only needs the aggregates
    (dict(block_column_include_aggregate=False, block_column_head_only=False), "include_aggregate"),   # so do deviations
    (dict(block_column_gain_init=-0.1), "non-negative"),
    (dict(block_column_trailing_layers=0), "at least 1"),
    (dict(block_column_blocks=[]), "attn_res_kimi"),
    (dict(block_column_blocks=[2]), "outside"),
    (dict(num_groups_per_token=[1, 1]), "attn_res_kimi"),                                    # no block has columns to keep
    (dict(block_residual_mode="attn_res_kimi"), "attn_res_column"),                         # column flags outside column mode
    (dict(residual_mode="attn_res"), "requires residual_mode='convex'"),
    (dict(residual_mode="attn_res_xblock"), "non-causal"),
    (dict(block_mlp_activations="swish"), "block_mlp_activations"),
    (dict(block_mlp_hidden_dims=[[256, 256]] * 2), "one hidden width"),
    (dict(block_layer_num_experts=[[1, 1]]), "one entry per block"),
    (dict(block_layer_num_experts=[[1], [1]]), "entries"),
    (dict(block_layer_num_experts=[[1, 0], [1]]), ">= 1"),
    (dict(block_layer_num_experts=[[1, 3], [1]], router_num_shared_experts=0), "at least two choices"),
    (dict(mlp_auto_dense_ratio=0.0), "positive"),
])
def test_configuration_rules_are_enforced(change, message):
    """Every rule the configuration variants come with is checked when the config is resolved, with a message that
    names the field (same constraints as the reference's expansion, nestor/backbones/nestor.py:2399-2600, 2785-2812)."""

    NestorConfig(**_COLUMN).resolve()
    with pytest.raises(ValueError, match=message):
        NestorConfig(**{**_COLUMN, **change}).resolve()


def test_block_specs_of_column_variants():
    """What ``resolve()`` derives for the column knobs: exports per block, merged prefixes, which blocks keep columns,
    and the widest read."""

    cfg = NestorConfig(**{**_COLUMN, "num_groups_per_token": [3, 2], "block_column_blocks": [0],
                          "block_column_trailing_layers": 1})
    a, b = cfg.resolve()
    assert (a.columns, a.exports, a.merged_prefix) == (True, 4, 1)        # 3 deviations + aggregate; first layer merged
    assert (b.columns, b.exports, b.merged_prefix) == (False, 1, 0)       # left out: one merged export
    assert cfg.max_depth_sources() == 1 + 4 + 1
    raw = NestorConfig(**{**_COLUMN, "num_groups_per_token": [3, 1], "block_column_include_aggregate": False,
                          "block_column_head_only": False, "block_column_deviation_sources": False}).resolve()
    assert [s.exports for s in raw] == [3, 1] and not raw[0].column_aggregate and not raw[0].column_deviation
    assert raw[1].column_aggregate is False                                 # a single column is its own aggregate
    sched = NestorConfig(**{**_COLUMN, "block_residual_mode": "attn_res_kimi", "num_groups": 1,
                            "num_groups_per_token": 1, "block_column_include_aggregate": False,
                            "block_column_head_only": False, "block_column_deviation_sources": False,
                            "block_layer_num_experts": [[4, 6], [5]], "router_num_shared_experts": [2, 5],
                            "router_num_experts_per_group_per_token": 2}).resolve()
    assert [sched[0].experts_of_layer(i) for i in range(2)] == [4, 6] and sched[0].bank_experts == 6
    assert sched[1].experts_of_layer(0) == 5
