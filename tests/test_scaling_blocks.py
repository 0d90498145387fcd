"""Role-typed building blocks: initialisation statistics, optimizer tags, and the arithmetic of each block."""

import math

import pytest
import torch

from nestor_b200.models.scaling import (
    GatedScaledMLP, RMSNorm, RoPE, ScaledEmbedding, ScaledLinear, ScaledMLP, convex_residual,
)
from nestor_b200.models.tags import get_tag
from nestor_b200.ops import reference as R


def test_roles_set_init_and_tags():
    torch.manual_seed(0)
    a = ScaledLinear(256, 64, role="in_stream", bias=True)
    assert abs(a.weight.std().item() - 1 / 16) < 0.01
    t = get_tag(a.weight)
    assert t.optimizer == "muon" and t.muon_scale == pytest.approx(0.5) and not get_tag(a.bias).weight_decay
    p = ScaledLinear(64, 256, role="projection", bias=False)
    sv = torch.linalg.svdvals(p.weight)
    assert torch.allclose(sv, torch.full_like(sv, 2.0), atol=1e-4)          # semi-orthogonal times sqrt(d_out/d_in)
    s = ScaledLinear(128, 8, role="score", bias=False, lr_mul=0.5)
    assert get_tag(s.weight).optimizer == "adamw" and get_tag(s.weight).lr_mul == pytest.approx(0.5 / 128)
    assert abs(s.weight.std().item() - 1 / 128) < 2e-3
    assert ScaledLinear(8, 1, role="score", bias=False, zero_init=True).weight.abs().sum() == 0
    with pytest.raises(ValueError, match="Unknown role"):
        ScaledLinear(4, 4, role="residual")


def test_mlp_blocks_norm_rope_and_residual():
    torch.manual_seed(1)
    mlp = ScaledMLP(16, [32], 4, out_role="score", bias=False)
    x = torch.randn(5, 16)
    assert torch.allclose(mlp(x), torch.nn.functional.gelu(x @ mlp.layers[0].weight.t()) @ mlp.layers[1].weight.t())
    assert get_tag(mlp.layers[0].weight).optimizer == "muon" and get_tag(mlp.layers[1].weight).optimizer == "adamw"
    g = GatedScaledMLP(16, 24)
    want = (torch.nn.functional.silu(x @ g.gate.weight.t()) * (x @ g.layers[0].weight.t())) @ g.layers[1].weight.t()
    assert g.gated and torch.allclose(g(x), want, atol=1e-6)
    n = RMSNorm(16, eps=1e-5)
    assert torch.allclose(n(x), R.rmsnorm(x, n.weight, 1e-5, torch.float32), atol=1e-6)
    assert RMSNorm(16, elementwise_affine=False).weight is None
    e = ScaledEmbedding(50, 16)
    assert get_tag(e.weight).optimizer == "adamw" and e(torch.tensor([[1, 2]])).shape == (1, 2, 16)
    rope = RoPE(8, base=100.0)
    q, pos = torch.randn(2, 6, 3, 8), torch.arange(6).repeat(2, 1)
    cos, sin = R.rope_tables(pos.reshape(-1), 8, 100.0)
    assert torch.allclose(rope(q, pos).reshape(12, 3, 8), R.apply_rope(q.reshape(12, 3, 8), cos, sin), atol=1e-6)
    assert torch.allclose(rope(q, pos).norm(dim=-1), q.norm(dim=-1), atol=1e-5)          # a rotation
    h, u = torch.randn(3, 4), torch.randn(3, 4)
    assert torch.allclose(convex_residual(h, u, 0.25), 0.75 * h + 0.25 * u)
    assert math.isclose(float(convex_residual(torch.ones(1), torch.zeros(1), 1 / 8)), 0.875)
