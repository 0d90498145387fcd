"""The two auxiliary router losses: our statement against the reference's own classes on the same router records, and
that a training forward of the model really feeds them (non-zero value, gradient reaching the router weights)."""

import sys
from pathlib import Path

import pytest
import torch

from nestor_b200.configs import ReferenceMoEAuxLossConfig, RouterBalanceLossConfig
from nestor_b200.train.losses import ReferenceMoEAuxLoss, RouterBalanceLoss

ROOT = Path(__file__).resolve().parent.parent


def _records(B=2, S=16):
    torch.manual_seed(0)
    mk = lambda C, k: {"scores": torch.randn(B, S, C, requires_grad=True),  # noqa: E731
                       "topk_indices": torch.randint(0, C, (B, S, k)),
                       "valid_token_mask": torch.rand(B, S) > 0.2}
    return {"blocks": [{"group_router": mk(8, 3), "layers": [{"expert_router": mk(6, 2)}, {"expert_router": mk(6, 2)}]},
                       {"group_router": mk(8, 4), "layers": [{"other": 1}]}]}


def test_aux_losses_match_reference_classes(monkeypatch):
    ref_root = ROOT / "baseline" / "_ref"
    if not (ref_root / "nestor").is_dir():
        pytest.skip("reference package not installed under baseline/_ref")
    monkeypatch.syspath_prepend(str(ref_root))
    try:
        from nestor.configs.losses import ReferenceMoEAuxLossConfig as RC2, RouterBalanceLossConfig as RC1
        from nestor.train.losses import ReferenceMoEAuxLoss as R2, RouterBalanceLoss as R1
    except Exception as exc:
        pytest.skip(f"reference import failed: {exc}")
    aux = _records()
    pred = torch.zeros(1)
    ours = RouterBalanceLoss(RouterBalanceLossConfig(balance_weight=0.3))(pred, pred, aux)
    theirs = R1(RC1(balance_weight=0.3))(pred, pred, aux)
    assert torch.allclose(ours.total, theirs.total, atol=1e-6)
    assert torch.allclose(ours.components["router_balance_group"], theirs.components["router_balance_group"], atol=1e-6)
    cfg = dict(coefficient=0.02, z_loss_weight=0.5)
    ours = ReferenceMoEAuxLoss(ReferenceMoEAuxLossConfig(**cfg))(pred, pred, aux)
    theirs = R2(RC2(**cfg))(pred, pred, aux)
    assert torch.allclose(ours.total, theirs.total, atol=1e-6)
    # flattened tokens (the layout our backbone reports) give the same value
    flat = {"blocks": [{"group_router": {k: v.reshape(-1, *v.shape[2:]) for k, v in b["group_router"].items()},
                        "layers": b["layers"]} for b in aux["blocks"]]}
    again = RouterBalanceLoss(RouterBalanceLossConfig(balance_weight=0.3))(pred, pred, flat)
    want = R1(RC1(balance_weight=0.3))(pred, pred, aux).components["router_balance_group"]
    assert torch.allclose(again.components["router_balance_group"], want, atol=1e-6)


@pytest.mark.parametrize("family", ["nestor", "moe"])
def test_model_feeds_the_aux_losses(family, tiny_scale):
    from nestor_b200.models import Model
    m = Model.from_config(tiny_scale.build_experiment(family, "tiny").jobs[0].model).train()
    ids = torch.randint(0, 100263, (2, 32))
    out = m(ids)
    bal = RouterBalanceLoss(RouterBalanceLossConfig(balance_weight=1.0))(out.pred, ids, out.aux)
    assert bal.total.item() > 0.5               # ~1 for a balanced router, never the dead zero
    if family == "nestor":
        bal.total.backward(retain_graph=True)
        g = m.backbone.blocks[0].group_router.score_mlp.layers[1].weight.grad
        assert g is not None and g.abs().sum() > 0
    else:
        ref = ReferenceMoEAuxLoss(ReferenceMoEAuxLossConfig(coefficient=0.01, z_loss_weight=0.001))(out.pred, ids, out.aux)
        assert ref.total.item() > 0
        ref.total.backward()
        g = m.backbone.blocks[0].layers[0].expert_router.score_mlp.layers[0].weight.grad
        assert g is not None and g.abs().sum() > 0


def test_packed_router_counts_sum_like_the_dictionaries():
    import torch

    from nestor_b200.models.nestor import RouterCounts, add_router_counts

    a = {"blocks.0.group_router": torch.tensor([3.0, 1.0, 4.0]), "blocks.0.layers.0.expert_router": torch.tensor([[1.0, 2.0], [3.0, 4.0]])}
    b = {k: v * 2 + 1 for k, v in a.items()}
    pa, pb = RouterCounts.pack(a), RouterCounts.pack(b)
    assert set(pa) == set(a) and all(torch.equal(pa[k], a[k]) and pa[k].shape == a[k].shape for k in a)
    total = add_router_counts(None, pa)
    assert total is not pa and torch.equal(total.flat, pa.flat)          # the first micro-batch's counts are copied
    total = add_router_counts(total, pb)
    pa.flat.zero_()                                                     # a replayed graph overwrites its static output
    for k in a:
        assert torch.equal(total[k], a[k] + b[k])
    plain = add_router_counts({}, a)
    plain = add_router_counts(plain, b)
    assert all(torch.equal(plain[k], total[k]) for k in a)
    assert add_router_counts(None, RouterCounts.pack({})) is not None
