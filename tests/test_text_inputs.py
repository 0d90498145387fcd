"""String inputs through the adapter's tokenizer and right-padded batches with a validity mask."""

import dataclasses as dc

import pytest
import torch

from nestor_b200.models.nestor import router_counts
from nestor_b200.train.losses import CausalLMLoss


def _byte_model(tiny_scale, family="nestor"):
    from nestor_b200.models import Model
    cfg = tiny_scale.build_experiment(family, "tiny").jobs[0].model
    cfg = dc.replace(cfg, adapter_config=dc.replace(cfg.adapter_config, tokenizer="bytes", max_length=40))
    torch.manual_seed(0)
    return Model.from_config(cfg).eval()


def test_padded_string_batch_equals_unpadded_sequences(tiny_scale):
    m = _byte_model(tiny_scale)
    texts = ["column routing keeps attention sparse", "short one"]
    with torch.no_grad():
        out = m(texts)
    ids, valid = m.adapter.encode_texts(texts)
    assert out.pred.shape[:2] == ids.shape and torch.equal(out.aux["valid_token_mask"], valid)
    assert valid[1].sum() == len(texts[1].encode()) and not bool(valid[1, -1])
    # padding behind a sequence does not change what the real tokens see
    for b, t in enumerate(texts):
        n = int(valid[b].sum())
        with torch.no_grad():
            alone = m(ids[b : b + 1, :n]).pred
        assert torch.allclose(out.pred[b, :n], alone[0], atol=1e-4, rtol=1e-4)
    # padding is neither a target nor a routing statistic
    loss = CausalLMLoss()(out.pred, ids, out.aux)
    n_targets = int(valid[:, 1:].sum())
    ref = torch.nn.functional.cross_entropy(out.pred[:, :-1].reshape(-1, out.pred.shape[-1]).float(),
                                            ids[:, 1:].masked_fill(~valid[:, 1:], -100).reshape(-1), ignore_index=-100)
    assert torch.allclose(loss.total, ref, atol=1e-5) and n_targets < ids[:, 1:].numel()
    counts = router_counts(m.backbone, out.aux)
    spec = m.backbone.blocks[0].spec
    assert int(counts["blocks.0.group_router"].sum()) == int(valid.sum()) * spec.k
    assert int(counts["blocks.0.layers.0.expert_pool.public_router"].sum()) == int(valid.sum()) * spec.k_p
    assert "valid_token_mask" in out.aux["blocks"][0]["group_router"]


def test_mask_must_be_a_prefix_and_tokenizer_errors_are_clear(tiny_scale):
    m = _byte_model(tiny_scale, "dense")
    ids = torch.randint(0, 255, (1, 6))
    with pytest.raises(ValueError, match="prefix"):
        m(ids, valid=torch.tensor([[True, False, True, True, False, False]]))
    assert m.adapter.tokenizer().decode(m.adapter.tokenizer().encode_ordinary("héllo")) == "héllo"


def test_adapter_norm_without_mup_and_head_hidden_layers(tiny_scale):
    """Without the reference-muP recipe the adapter normalises embeddings to unit RMS (reference
    nestor/adapters/text.py:150); a head with hidden_dims runs its hidden layers in front of the vocabulary matrix,
    and the fused head + cross-entropy path sees the same features as the plain one."""

    from nestor_b200.models import Model
    cfg = tiny_scale.build_experiment("dense", "tiny").jobs[0].model
    cfg = dc.replace(cfg, reference_mup=None,
                     head_config=dc.replace(cfg.head_config, hidden_dims=[48], activation="gelu"))
    torch.manual_seed(0)
    m = Model.from_config(cfg).eval()
    ids = torch.randint(0, 255, (2, 12))
    x = m.adapter(ids)
    assert torch.allclose(x.pow(2).mean(-1), torch.ones(2, 12), atol=1e-3)
    assert m.adapter.norm is not None and len(m.head.hidden) == 1 and m.head.weight.shape[1] == 48
    with torch.no_grad():
        plain = m(ids)
        m.fused_head = True
        fused = m(ids)
    assert fused.pred.shape[-1] == 48 and plain.pred.shape[-1] == cfg.head_config.vocab_size
    a = CausalLMLoss()(plain.pred, ids, plain.aux).total
    b = CausalLMLoss()(fused.pred, ids, fused.aux).total
    assert torch.allclose(a, b, atol=1e-5)
    # the hidden layer is an in-stream matrix (Muon) and trains
    names = {n for n, _ in m.named_parameters()}
    assert "head.hidden.0.weight" in names and "adapter.norm.weight" in names
