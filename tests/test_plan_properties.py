"""Property tests (random shapes) of the dispatch plans and the routing op: the invariants the kernels rely on hold for
every batch size, sequence length, column count and top-k, including positions handed in explicitly."""

import torch
from hypothesis import given, settings, strategies as st

from nestor_b200.ops import reference as R

_shapes = st.tuples(st.integers(1, 4), st.integers(1, 33), st.integers(1, 9)).flatmap(
    lambda t: st.tuples(st.just(t[0]), st.just(t[1]), st.just(t[2]), st.integers(1, t[2]), st.integers(0, 2**31 - 1)))


@settings(max_examples=40, deadline=None, derandomize=True)
@given(_shapes)
def test_column_plan_invariants(shape):
    B, S, G, k, seed = shape
    g = torch.Generator().manual_seed(seed)
    idx = torch.rand(B, S, G, generator=g).topk(k, dim=-1).indices
    plan = R.build_column_plan(idx, G)
    rows = B * S * k
    tok, slot = plan.tok_of_row.long(), plan.slot_of_row.long()
    assert plan.rows == rows and plan.k == k and plan.G == G
    assert torch.equal(plan.row_of_slot.long()[tok, slot], torch.arange(rows))          # inverse maps agree
    assert sorted(plan.row_of_slot.reshape(-1).tolist()) == list(range(rows))            # bijection
    seg = plan.seg_start.long()
    assert seg[0] == 0 and seg[-1] == rows and len(seg) == G * B + 1 and (seg[1:] >= seg[:-1]).all()
    # every row sits in the segment of (its column, its sequence), in token order inside the segment
    col = idx.reshape(B * S, k)[tok, slot]
    want_segment = col * B + tok // S
    got_segment = torch.searchsorted(seg, torch.arange(rows), right=True) - 1
    assert torch.equal(got_segment, want_segment)
    same = got_segment[1:] == got_segment[:-1]
    assert (tok[1:][same] > tok[:-1][same]).all()
    assert torch.equal(plan.pos_of_row.long(), tok % S)
    assert torch.equal(plan.col_start.long(), seg[::B])


@settings(max_examples=25, deadline=None, derandomize=True)
@given(_shapes)
def test_column_plan_carries_explicit_positions(shape):
    B, S, G, k, seed = shape
    g = torch.Generator().manual_seed(seed)
    idx = torch.rand(B, S, G, generator=g).topk(k, dim=-1).indices
    pos = torch.randint(0, 5000, (B, S), generator=g)
    plan = R.build_column_plan(idx, G, pos)
    assert torch.equal(plan.pos_of_row.long(), pos.reshape(-1)[plan.tok_of_row.long()])


@settings(max_examples=40, deadline=None, derandomize=True)
@given(st.integers(1, 60), st.integers(1, 4), st.integers(1, 12), st.integers(0, 2**31 - 1))
def test_expert_plan_invariants(T, slots, E, seed):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, E, (T, slots), generator=g)
    plan = R.build_expert_plan(ids, E)
    flat = ids.reshape(-1)
    order, inv, off = plan.order.long(), plan.inv.long(), plan.offsets.long()
    assert plan.n == T * slots and plan.slots == slots and plan.E == E
    assert torch.equal(inv[order], torch.arange(flat.numel())) and torch.equal(order[inv], torch.arange(flat.numel()))
    assert off[0] == 0 and off[-1] == flat.numel() and torch.equal(off.diff(), torch.bincount(flat, minlength=E))
    sorted_ids = flat[order]
    assert (sorted_ids[1:] >= sorted_ids[:-1]).all()
    same = sorted_ids[1:] == sorted_ids[:-1]
    assert (order[1:][same] > order[:-1][same]).all()                                   # stable inside an expert


@settings(max_examples=40, deadline=None, derandomize=True)
@given(st.integers(1, 40), st.integers(1, 10), st.integers(0, 2**31 - 1), st.sampled_from(["renorm", "switch"]))
def test_routing_invariants(T, C, seed, mode):
    g = torch.Generator().manual_seed(seed)
    k = int(torch.randint(1, C + 1, (1,), generator=g))
    scores, bias = torch.randn(T, C, generator=g), torch.randn(C, generator=g)
    idx, gates = R.route_topk(scores, bias, k, mode)
    assert idx.shape == gates.shape == (T, k)
    assert all(len(set(row)) == k for row in idx.tolist())                               # k distinct choices
    assert torch.equal(idx.sort(-1).values, (scores + bias).topk(k).indices.sort(-1).values)   # the bias only selects
    if mode == "renorm":
        assert torch.allclose(gates.sum(-1), torch.ones(T), atol=1e-5)
        assert torch.allclose(gates, torch.softmax(scores.gather(-1, idx), -1), atol=1e-6)
    else:
        assert torch.allclose(gates, torch.softmax(scores, -1).gather(-1, idx), atol=1e-6)
        assert (gates.sum(-1) <= 1 + 1e-5).all()


@settings(max_examples=12, deadline=None, derandomize=True)
@given(st.integers(1, 3), st.integers(1, 17), st.integers(1, 5), st.integers(0, 2**31 - 1), st.booleans())
def test_column_attention_against_the_masked_definition(B, S, G, seed, causal):
    """Column attention over the packed plan equals the definition written with dense masks: token ``t`` attends, in
    column ``c``, to the members of ``c`` in its own sequence (only earlier ones and itself when causal)."""

    g = torch.Generator().manual_seed(seed)
    k = int(torch.randint(1, G + 1, (1,), generator=g))
    H, hd, d = 2, 4, 12
    n = torch.randn(B * S, d, generator=g)
    idx = torch.rand(B, S, G, generator=g).topk(k, -1).indices
    gates = torch.rand(B * S, k, generator=g)
    wqkv = torch.randn(G, 3 * H * hd, d, generator=g) * 0.3
    wo = torch.randn(G, d, H * hd, generator=g) * 0.3
    plan = R.build_column_plan(idx, G)
    got = R.column_attention(n, plan, gates, wqkv, wo, H, hd, 10000.0, torch.float32, causal=causal)
    cos, sin = R.rope_tables(torch.arange(S).repeat(B), hd, 10000.0)
    flat = idx.reshape(B * S, k)
    want = torch.zeros(B * S, k, d)
    inner = H * hd
    for c in range(G):
        qkv = n @ wqkv[c].t()
        q = R.apply_rope(qkv[:, :inner].reshape(-1, H, hd), cos, sin)
        kk = R.apply_rope(qkv[:, inner:2 * inner].reshape(-1, H, hd), cos, sin)
        v = qkv[:, 2 * inner:].reshape(-1, H, hd)
        member = (flat == c).any(-1)                                                      # [T]
        for b in range(B):
            rows = torch.arange(b * S, (b + 1) * S)
            m = member[rows]
            if not m.any():
                continue
            sc = torch.einsum("thd,shd->hts", q[rows], kk[rows]) / hd
            mask = m.unsqueeze(0) & m.unsqueeze(1)                                        # members see members
            if causal:
                mask = mask & torch.ones(S, S, dtype=torch.bool).tril()
            p = torch.softmax(sc.masked_fill(~mask, float("-inf")), dim=-1).nan_to_num(0.0)
            o = torch.einsum("hts,shd->thd", p, v[rows]).reshape(S, inner) @ wo[c].t()
            for j in range(k):
                sel = flat[rows, j] == c
                want[rows[sel], j] = o[sel] * gates[rows[sel], j].unsqueeze(-1)
    assert torch.allclose(got, want, atol=2e-4), float((got - want).abs().max())


@settings(max_examples=20, deadline=None, derandomize=True)
@given(st.integers(1, 20), st.integers(1, 6), st.sampled_from([1, 2, 3]), st.integers(0, 2**31 - 1),
       st.sampled_from(["swiglu", "gelu", "relu", "tanh"]))
def test_expert_bank_against_a_per_token_loop(T, E, group, seed, activation):
    g = torch.Generator().manual_seed(seed)
    d, h = 6, 5
    slots = group * int(torch.randint(1, 3, (1,), generator=g))
    x = torch.randn(T, d, generator=g)
    ids = torch.randint(0, E, (T, slots), generator=g)
    w = torch.rand(T, slots, generator=g)
    wu, wg, wd = (torch.randn(*s, generator=g) * 0.4 for s in ((E, d, h), (E, d, h), (E, h, d)))
    gated = activation == "swiglu"
    got = R.expert_bank(x, R.build_expert_plan(ids, E), w, wu, wg if gated else None, wd, torch.float32, group, activation)
    want = torch.zeros(T, slots // group, d)
    for t in range(T):
        for s in range(slots):
            e = ids[t, s]
            up = x[t] @ wu[e]
            hid = torch.nn.functional.silu(x[t] @ wg[e]) * up if gated else R.POINTWISE_ACTIVATIONS[activation](up)
            want[t, s // group] += w[t, s] * (hid @ wd[e])
    assert torch.allclose(got, want, atol=1e-5)


@settings(max_examples=25, deadline=None, derandomize=True)
@given(st.integers(1, 12), st.integers(1, 6), st.integers(1, 9), st.integers(0, 2**31 - 1), st.booleans())
def test_depth_read_and_stream_identities(T, k, n_src, seed, per_source):
    g = torch.Generator().manual_seed(seed)
    d = 8
    srcs = [torch.randn(T, d, generator=g) * float(torch.rand((), generator=g) * 3 + 0.1) for _ in range(n_src)]
    q = torch.randn(n_src, d, generator=g) if per_source else torch.randn(d, generator=g)
    gains = torch.rand(n_src + 2, generator=g) + 0.5
    out = R.depth_read(srcs, q, gains)
    r = [torch.rsqrt(s.pow(2).mean(-1) + 1e-6) for s in srcs]
    z = torch.stack([ri * (s @ (q[i] if per_source else q)) for i, (s, ri) in enumerate(zip(srcs, r))], -1) / d ** 0.5
    w = torch.softmax(z, -1) * gains[:n_src]
    want = sum((w[:, i] * r[i]).unsqueeze(-1) * srcs[i] for i in range(n_src))
    assert torch.allclose(out, want, atol=1e-5)
    # rescaling a source changes nothing (unit-RMS keys and values), up to the epsilon floor
    scaled = [s * 7.0 for s in srcs]
    assert torch.allclose(R.depth_read(scaled, q, gains), out, atol=1e-3, rtol=1e-3)
    # a zero query is the gain-weighted mean of the unit-RMS sources
    zero = R.depth_read(srcs, torch.zeros_like(q), gains)
    assert torch.allclose(zero, sum((gains[i] / n_src * r[i]).unsqueeze(-1) * srcs[i] for i in range(n_src)), atol=1e-5)
    # the cache only removes repeated work
    cache = R.DepthKeyCache(srcs[: max(1, n_src - 1)])
    assert torch.equal(R.depth_read(srcs, q, gains, key_cache=cache), out)

    # block exit: deviations sum to zero, the aggregate is the mean; layer_combine adds one update to both states
    streams = torch.randn(T, k, d, generator=g)
    dev, agg = R.block_exit(streams)
    assert dev.shape == (k, T, d) and torch.allclose(dev.sum(0), torch.zeros(T, d), atol=1e-5)
    assert torch.allclose(agg, streams.mean(1), atol=1e-6)
    attn, pub = torch.randn(T, k, d, generator=g), torch.randn(T, d, generator=g)
    priv, path = torch.randn(T, k, d, generator=g), torch.softmax(torch.randn(T, 2, generator=g), -1)
    new_streams, running = R.layer_combine(attn, priv, pub, path, streams, streams.mean(1), torch.float32)
    update = attn + path[:, 1:2].unsqueeze(-1) * priv + (path[:, 0:1] * pub).unsqueeze(1)
    assert torch.allclose(new_streams, streams + update, atol=1e-5)
    assert torch.allclose(running, new_streams.mean(1), atol=1e-5)                       # the running mean stays the mean
    assert torch.allclose(R.mid_source(streams.mean(1), attn), (streams + attn).mean(1), atol=1e-5)


@settings(max_examples=20, deadline=None, derandomize=True)
@given(st.integers(1, 40), st.integers(2, 30), st.integers(1, 16), st.integers(0, 2**31 - 1))
def test_chunked_head_loss_is_the_full_cross_entropy(T, V, chunk, seed):
    g = torch.Generator().manual_seed(seed)
    d = 6
    h = torch.randn(T, d, generator=g, requires_grad=True)
    w = torch.randn(V, d, generator=g, requires_grad=True)
    tg = torch.randint(0, V, (T,), generator=g)
    tg[torch.rand(T, generator=g) < 0.3] = -100                      # ignored positions (padding, the last token)
    ls, cnt = R.lm_head_ce(h, w, tg, 0.25, torch.float32, chunk_rows=chunk)
    want = torch.nn.functional.cross_entropy((h @ w.t()) * 0.25, tg, ignore_index=-100, reduction="sum")
    assert int(cnt) == int((tg != -100).sum())
    assert torch.allclose(ls, want, atol=1e-4)
    if int(cnt):
        g1 = torch.autograd.grad(ls, [h, w])
        g2 = torch.autograd.grad(want, [h, w])
        assert all(torch.allclose(a, b, atol=1e-5) for a, b in zip(g1, g2))


@settings(max_examples=15, deadline=None, derandomize=True)
@given(st.integers(2, 24), st.integers(2, 24), st.integers(1, 3), st.integers(0, 2**31 - 1))
def test_newton_schulz_contracts_the_spread_of_singular_values(rows, cols, batch, seed):
    """Five quintic steps move every singular value of a (batch of) matrices into a band around one, for wide, tall
    and square shapes alike (the update direction Muon applies)."""

    g = torch.Generator().manual_seed(seed)
    m = torch.randn(batch, rows, cols, generator=g)
    out = R.newton_schulz(m, steps=5).float()
    assert out.shape == m.shape and torch.isfinite(out).all()
    sv = torch.linalg.svdvals(out)
    k = min(rows, cols)
    assert sv.shape[-1] == k and float(sv.max()) < 1.35
    assert float(sv.median()) > 0.3                                   # the bulk has been lifted towards one
