"""Depth key cache (bit-identical reads, fewer scale reductions) and the per-source block attention residual."""

import torch

from nestor_b200 import ops
from nestor_b200.models.modules import BlockAttentionResidual
from nestor_b200.ops import reference as R


def test_key_cache_is_exact_and_lazy():
    torch.manual_seed(0)
    T, d = 12, 32
    fixed = [torch.randn(T, d) for _ in range(3)]
    q, gains = torch.randn(d) * 0.3, torch.rand(8) + 0.5
    cache = R.DepthKeyCache(fixed[:2], eps=1e-6)
    tail = torch.randn(T, d)
    a = R.depth_read([*fixed[:2], tail], q, gains, 1e-6, key_cache=cache)
    b = R.depth_read([*fixed[:2], tail], q, gains, 1e-6)
    assert torch.equal(a, b) and cache.computed == 2
    cache.extend([fixed[2]])
    c = R.depth_read([*fixed, tail], q, gains, 1e-6, key_cache=cache)
    assert torch.equal(c, R.depth_read([*fixed, tail], q, gains, 1e-6)) and cache.computed == 3    # only the new source
    import pytest
    with pytest.raises(ValueError, match="own tensors"):
        R.depth_read([fixed[0].clone(), fixed[1], fixed[2]], q, gains, 1e-6, key_cache=cache)
    with pytest.raises(ValueError, match="epsilon"):
        R.depth_read(fixed, q, gains, 1e-5, key_cache=cache)


def test_model_forward_shares_scales_and_matches_uncached(tiny_scale, monkeypatch):
    from nestor_b200.models import Model
    torch.manual_seed(0)
    m = Model.from_config(tiny_scale.build_experiment("nestor", "tiny").jobs[0].model).eval()
    with torch.no_grad():
        for n, p in m.named_parameters():
            if "query" in n:
                p.normal_(0, 0.5)
    ids = torch.randint(0, 100263, (2, 32))
    with torch.no_grad():
        cached = m(ids).pred
    kc = m.backbone.last_key_cache
    blocks = len(m.backbone.blocks)
    assert kc is not None and kc.num_sources == blocks + 1 and kc.computed == blocks      # the last aggregate is never re-read
    reads = 2 * sum(len(b.layers) for b in m.backbone.blocks)
    assert kc.computed < reads                      # without the cache every read reduces every source again
    monkeypatch.setenv("NESTOR_NO_DEPTH_KEY_CACHE", "1")
    with torch.no_grad():
        plain = m(ids).pred
    assert m.backbone.last_key_cache is None and torch.equal(cached, plain)


def test_block_attention_residual_equation_and_zero_query_mean():
    torch.manual_seed(1)
    bar = BlockAttentionResidual([16, 16, 24], 16, std=0.2)
    srcs = [torch.randn(2, 5, 16), torch.randn(2, 5, 16), torch.randn(2, 5, 24)]
    vals = [s @ v.weight.t() for s, v in zip(srcs, bar.value_projections)]
    assert torch.allclose(bar(srcs), sum(vals) / 3, atol=1e-6)            # zero query: plain mean of the values
    with torch.no_grad():
        bar.query.weight.normal_(0, 1.0)
    keys = [s @ k.weight.t() for s, k in zip(srcs, bar.key_projections)]
    logits = torch.stack([(k @ bar.query.weight.t()).squeeze(-1) for k in keys])
    want = (torch.stack(vals) * logits.softmax(0).unsqueeze(-1)).sum(0)
    assert torch.allclose(bar(srcs), want, atol=1e-6)
    names = dict(bar.named_parameters())
    assert {"key_projections.0.weight", "value_projections.2.weight", "query.weight"} <= set(names)
    from nestor_b200.models.tags import get_tag
    assert get_tag(names["query.weight"]).optimizer == "adamw" and get_tag(names["key_projections.0.weight"]).optimizer == "muon"
