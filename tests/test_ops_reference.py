"""The PyTorch oracle ops against slow, obviously-correct restatements of the equations."""

import math

import pytest
import torch
import torch.nn.functional as F

from nestor_b200.ops import reference as R


def test_column_plan_is_a_bijection_with_ordered_segments():
    torch.manual_seed(0)
    B, S, G, k = 3, 37, 5, 2
    idx = torch.rand(B, S, G).topk(k, dim=-1).indices
    plan = R.build_column_plan(idx, G)
    rows = B * S * k
    assert plan.rows == rows
    assert sorted(plan.row_of_slot.reshape(-1).tolist()) == list(range(rows))          # bijection
    tok, slot = plan.tok_of_row.long(), plan.slot_of_row.long()
    assert torch.equal(plan.row_of_slot.long()[tok, slot], torch.arange(rows))        # inverse maps agree
    seg = plan.seg_start.tolist()
    assert seg[0] == 0 and seg[-1] == rows and len(seg) == G * B + 1
    col_of_row = plan.idx.long()[tok, slot]
    for c in range(G):
        for b in range(B):
            a, e = seg[c * B + b], seg[c * B + b + 1]
            assert (col_of_row[a:e] == c).all()
            t = tok[a:e]
            assert ((t // S) == b).all() and (t[1:] > t[:-1]).all()                    # one sequence, token order
            assert torch.equal(plan.pos_of_row[a:e].long(), t % S)
    assert torch.equal(plan.col_start, plan.seg_start[::B])


def test_expert_plan_groups_rows_stably():
    torch.manual_seed(1)
    ids = torch.randint(0, 7, (50, 3))
    plan = R.build_expert_plan(ids, 7)
    flat = ids.reshape(-1)
    sorted_ids = flat[plan.order.long()]
    assert (sorted_ids[1:] >= sorted_ids[:-1]).all()
    off = plan.offsets.tolist()
    for e in range(7):
        seg = plan.order[off[e]:off[e + 1]].long()
        assert (flat[seg] == e).all() and (seg[1:] > seg[:-1]).all()                   # stable inside an expert
    assert torch.equal(plan.inv.long()[plan.order.long()], torch.arange(flat.numel()))


def test_route_topk_gate_modes():
    torch.manual_seed(2)
    scores, bias = torch.randn(11, 6), torch.randn(6) * 0.1
    idx, gates = R.route_topk(scores, bias, 3, "renorm")
    assert torch.equal(idx, (scores + bias).topk(3).indices)
    assert torch.allclose(gates.sum(-1), torch.ones(11), atol=1e-6)
    assert torch.allclose(gates, torch.softmax(scores.gather(-1, idx), -1))
    idx2, sw = R.route_topk(scores, bias, 2, "switch")
    assert torch.allclose(sw, torch.softmax(scores, -1).gather(-1, idx2)) and (sw.sum(-1) < 1).all()


def test_routing_tape_replays_selections():
    torch.manual_seed(3)
    tape = R.RoutingTape()
    s1, s2 = torch.randn(5, 4), torch.randn(5, 4)
    R.set_routing_tape(tape, "record")
    a, _ = R.route_topk(s1, torch.zeros(4), 2, "renorm")
    R.set_routing_tape(tape, "replay")
    b, g = R.route_topk(s2, torch.zeros(4), 2, "renorm")
    R.set_routing_tape(None)
    assert torch.equal(a, b) and torch.allclose(g, torch.softmax(s2.gather(-1, a), -1))


def test_depth_read_matches_the_equation_and_is_uniform_at_zero_query():
    torch.manual_seed(4)
    d, n = 16, 4
    srcs = [torch.randn(7, d) * (i + 1) for i in range(n)]
    q, gains = torch.randn(d), torch.rand(6) + 0.5
    out = R.depth_read(srcs, q, gains, 1e-6)
    keys = [s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + 1e-6) for s in srcs]
    z = torch.stack([(k * q).sum(-1) for k in keys], -1) / math.sqrt(d)
    w = torch.softmax(z, -1)
    want = sum(w[:, i:i + 1] * gains[i] * keys[i] for i in range(n))
    assert torch.allclose(out, want, atol=1e-5)
    uni = R.depth_read(srcs, torch.zeros(d), torch.ones(6))
    assert torch.allclose(uni, sum(keys) / n, atol=1e-5)


def test_rmsnorm_and_rope():
    torch.manual_seed(5)
    x, w = torch.randn(5, 12), torch.rand(12)
    y = R.rmsnorm(x, w, 1e-5, torch.float32)
    assert torch.allclose(y, x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5) * w, atol=1e-6)
    pos = torch.arange(9)
    cos, sin = R.rope_tables(pos, 8, 10000.0)
    v = torch.randn(9, 2, 8)
    r = R.apply_rope(v, cos, sin)
    assert torch.allclose(r.norm(dim=-1), v.norm(dim=-1), atol=1e-5)                   # a rotation
    assert torch.allclose(r[0], v[0], atol=1e-6)                                       # position 0 is the identity
    # relative-position property: <rope(q, m), rope(k, n)> depends on m - n only
    q, k = torch.randn(1, 1, 8), torch.randn(1, 1, 8)
    def dot(m, n):
        cm, sm = R.rope_tables(torch.tensor([m]), 8, 10000.0); cn, sn = R.rope_tables(torch.tensor([n]), 8, 10000.0)
        return (R.apply_rope(q, cm, sm) * R.apply_rope(k, cn, sn)).sum()
    assert torch.allclose(dot(5, 2), dot(9, 6), atol=1e-5)


def _naive_column_attention(n, idx, gates, wqkv, wo, B, S, G, H, hd, base):
    """Masked full attention per column: the definition, O(G S^2)."""
    T, d = n.shape
    k = idx.shape[1]
    inner = H * hd
    out = torch.zeros(T, k, d)
    pos = torch.arange(S).repeat(B)
    cos, sin = R.rope_tables(pos, hd, base)
    for c in range(G):
        qkv = n @ wqkv[c].t()
        q = R.apply_rope(qkv[:, :inner].reshape(T, H, hd), cos, sin)
        kk = R.apply_rope(qkv[:, inner:2 * inner].reshape(T, H, hd), cos, sin)
        v = qkv[:, 2 * inner:].reshape(T, H, hd)
        member = (idx == c).any(-1)
        for b in range(B):
            sl = slice(b * S, (b + 1) * S)
            m = member[sl]
            if not m.any():
                continue
            qq, kb, vb = q[sl][m].transpose(0, 1), kk[sl][m].transpose(0, 1), v[sl][m].transpose(0, 1)
            L = qq.shape[1]
            s = (qq @ kb.transpose(1, 2)) / hd
            s = s.masked_fill(~torch.ones(L, L, dtype=torch.bool).tril(), float("-inf"))
            o = (torch.softmax(s, -1) @ vb).transpose(0, 1).reshape(L, inner) @ wo[c].t()
            toks = torch.arange(b * S, (b + 1) * S)[m]
            for j in range(k):
                sel = idx[toks, j] == c
                out[toks[sel], j] = o[sel] * gates[toks[sel], j:j + 1]
    return out


def test_column_attention_matches_masked_definition():
    torch.manual_seed(6)
    B, S, G, k, H, hd, d = 2, 19, 4, 2, 2, 8, 24
    n = torch.randn(B * S, d)
    idx = torch.rand(B, S, G).topk(k, -1).indices
    gates = torch.rand(B * S, k)
    wqkv, wo = torch.randn(G, 3 * H * hd, d) * 0.2, torch.randn(G, d, H * hd) * 0.2
    plan = R.build_column_plan(idx, G)
    got = R.column_attention(n, plan, gates, wqkv, wo, H, hd, 10000.0, torch.float32)
    want = _naive_column_attention(n, idx.reshape(B * S, k), gates, wqkv, wo, B, S, G, H, hd, 10000.0)
    assert torch.allclose(got, want, atol=1e-4)


def test_expert_bank_matches_per_token_loop():
    torch.manual_seed(7)
    T, d, E, h, slots, group = 13, 12, 5, 8, 4, 2
    x = torch.randn(T, d)
    ids, w = torch.randint(0, E, (T, slots)), torch.rand(T, slots)
    wu, wg, wd = torch.randn(E, d, h) * 0.3, torch.randn(E, d, h) * 0.3, torch.randn(E, h, d) * 0.3
    got = R.expert_bank(x, R.build_expert_plan(ids, E), w, wu, wg, wd, torch.float32, group)
    want = torch.zeros(T, slots // group, d)
    for t in range(T):
        for s in range(slots):
            e = ids[t, s]
            want[t, s // group] += w[t, s] * ((F.silu(x[t] @ wg[e]) * (x[t] @ wu[e])) @ wd[e])
    assert torch.allclose(got, want, atol=1e-5)


def test_lm_head_ce_chunks_agree_with_full_cross_entropy():
    torch.manual_seed(8)
    T, d, V = 37, 10, 53
    h, w = torch.randn(T, d, requires_grad=True), torch.randn(V, d, requires_grad=True)
    tg = torch.randint(0, V, (T,)); tg[::5] = -100
    ls, cnt = R.lm_head_ce(h, w, tg, 0.125, torch.float32, chunk_rows=8)
    want = F.cross_entropy((h @ w.t()) * 0.125, tg, ignore_index=-100, reduction="sum")
    assert torch.allclose(ls, want, atol=1e-4) and int(cnt) == int((tg != -100).sum())
    g1 = torch.autograd.grad(ls, [h, w]); g2 = torch.autograd.grad(want, [h, w])
    assert all(torch.allclose(a, b, atol=1e-5) for a, b in zip(g1, g2))


def test_newton_schulz_pushes_singular_values_toward_one():
    torch.manual_seed(9)
    for shape in [(24, 40), (40, 24), (3, 16, 16)]:
        g = torch.randn(*shape)
        o = R.newton_schulz(g, 5).float()
        sv = torch.linalg.svdvals(o)
        assert sv.max() < 1.35 and sv.min() > 0.3, (shape, sv.min().item(), sv.max().item())
        assert o.shape == g.shape


def test_stream_ops_are_consistent():
    torch.manual_seed(10)
    T, k, d = 6, 3, 8
    attn, priv, pub, path = torch.randn(T, k, d), torch.randn(T, k, d), torch.randn(T, d), torch.softmax(torch.randn(T, 2), -1)
    s0, r0 = R.layer_combine(attn, priv, pub, path, None, None, torch.float32)
    assert torch.allclose(r0, s0.mean(1), atol=1e-6)
    s1, r1 = R.layer_combine(attn, priv, pub, path, s0, r0, torch.float32)
    assert torch.allclose(s1, 2 * s0, atol=1e-6) and torch.allclose(r1, s1.mean(1), atol=1e-6)
    assert torch.allclose(R.mid_source(r0, attn), r0 + attn.mean(1))
    dev, agg = R.block_exit(s1)
    assert dev.shape == (k, T, d) and torch.allclose(dev.sum(0), torch.zeros(T, d), atol=1e-5)
    assert torch.allclose(dev[1] + agg, s1[:, 1], atol=1e-6)
