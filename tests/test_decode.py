"""Incremental decoding with the key/value cache reproduces the full-sequence forward token by token."""

import pytest
import torch


@pytest.mark.parametrize("family", ["nestor", "moe", "dense"])
def test_stepwise_decode_matches_full_forward(family, tiny_scale):
    from nestor_b200.models import Model
    torch.manual_seed(0)
    m = Model.from_config(tiny_scale.build_experiment(family, "tiny").jobs[0].model).eval()
    with torch.no_grad():
        for n, p in m.named_parameters():          # make the depth reads non-trivial
            if "query" in n:
                p.normal_(0, 0.5)
            if "value_gains" in n:
                p.uniform_(0.5, 1.5)
    B, S = 2, 24
    ids = torch.randint(0, 100263, (B, S))
    with torch.no_grad():
        full = m(ids).pred.float()                                  # [B, S, V]
    cache = m.init_kv_cache(B, S)
    for t in range(S):
        step = m.decode_step(ids[:, t], cache)
        assert torch.allclose(step, full[:, t], atol=2e-4, rtol=1e-4), (family, t, (step - full[:, t]).abs().max())
    assert cache.length == S
    # a token enters only the columns it was routed to
    blk = m.backbone.blocks[0]
    counts = cache.blocks[0][0].count
    assert int(counts.sum()) == B * S * blk.spec.k and int(counts.max()) <= S


@pytest.mark.parametrize("head_only", [True, False])
def test_stepwise_decode_through_merged_blocks_and_trailing_windows(head_only, tiny_scale):
    """Blocks left out of ``block_column_blocks`` (merged recurrence) and blocks whose leading layers are merged
    (``block_column_trailing_layers``) decode token by token to the same logits as the full forward, with narrow
    and with column-resolved sublayer reads."""

    import dataclasses as dc
    from nestor_b200.models import Model
    torch.manual_seed(2)
    cfg = tiny_scale.build_experiment("nestor", "tiny").jobs[0].model
    cfg = dc.replace(cfg, backbone_config=dc.replace(cfg.backbone_config, block_column_blocks=[0, 3],
                                                     block_column_trailing_layers=1,
                                                     block_column_head_only=head_only,
                                                     block_column_head_query_per_source=True))
    m = Model.from_config(cfg).eval()
    with torch.no_grad():
        for n, p in m.named_parameters():
            if "query" in n:
                p.normal_(0, 0.5)
            if "value_gains" in n:
                p.uniform_(0.5, 1.5)
    B, S = 2, 16
    ids = torch.randint(0, 100263, (B, S))
    with torch.no_grad():
        full = m(ids).pred.float()
    cache = m.init_kv_cache(B, S)
    for t in range(S):
        step = m.decode_step(ids[:, t], cache)
        assert torch.allclose(step, full[:, t], atol=2e-4, rtol=1e-4), (t, (step - full[:, t]).abs().max())


def test_generate_is_greedy_continuation(tiny_scale):
    from nestor_b200.models import Model
    torch.manual_seed(1)
    m = Model.from_config(tiny_scale.build_experiment("nestor", "tiny").jobs[0].model).eval()
    prompt = torch.randint(0, 100263, (2, 5))
    out = m.generate(prompt, 4)
    assert out.shape == (2, 9) and torch.equal(out[:, :5], prompt)
    with torch.no_grad():
        nxt = m(out[:, :8]).pred[:, -1].argmax(-1)
    assert torch.equal(nxt, out[:, 8])
    with pytest.raises(ValueError, match="cache"):
        cache = m.init_kv_cache(2, 2)
        for t in range(3):
            m.decode_step(prompt[:, t], cache)


def test_stepwise_decode_with_within_block_history_attention(tiny_scale):
    """``residual_mode='attn_res'`` mixes a token's own sublayer history, so it decodes token by token as well."""

    import dataclasses as dc
    from nestor_b200.models import Model
    torch.manual_seed(3)
    cfg = tiny_scale.build_experiment("moe", "tiny").jobs[0].model
    cfg = dc.replace(cfg, backbone_config=dc.replace(cfg.backbone_config, residual_mode="attn_res",
                                                     block_residual_mode="attn_res"))
    m = Model.from_config(cfg).eval()
    with torch.no_grad():
        for n, p in m.named_parameters():
            if "query" in n:
                p.normal_(0, 0.1)
    B, S = 2, 12
    ids = torch.randint(0, 100263, (B, S))
    with torch.no_grad():
        full = m(ids).pred.float()
    cache = m.init_kv_cache(B, S)
    for t in range(S):
        step = m.decode_step(ids[:, t], cache)
        assert torch.allclose(step, full[:, t], atol=2e-4, rtol=1e-4), (t, (step - full[:, t]).abs().max())
