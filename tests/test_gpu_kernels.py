"""sm_100a kernels against plain PyTorch fp32 references (run with ``-m gpu`` on a B200).

Outputs are pre-filled with NaN so any row or column a kernel fails to write shows up; grouped cases
include empty groups, ragged tiles and widths that are not multiples of the tile sizes.
"""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def _offsets(rows, groups, empty=()):
    w = torch.rand(groups)
    for e in empty:
        w[e] = 0
    c = (w / w.sum() * rows).floor().long()
    c[-1] += rows - c.sum()
    off = torch.zeros(groups + 1, dtype=torch.int32)
    off[1:] = c.cumsum(0)
    return off.cuda()


@pytest.fixture(autouse=True)
def _status():
    from nestor_b200.ops import _lib
    yield
    torch.cuda.synchronize()
    _lib.check_status(torch.device("cuda"))


@pytest.mark.parametrize("M,N,K", [(256, 128, 64), (1000, 600, 640), (4096, 256, 200), (333, 72, 80)])
def test_gemm_single_group(M, N, K):
    from nestor_b200.ops import gemm as G
    torch.manual_seed(0)
    A, B = torch.randn(M, K, device="cuda").to(BF), torch.randn(N, K, device="cuda").to(BF)
    out = torch.full((M, N), float("nan"), device="cuda", dtype=BF)
    G.gemm_rows(A, B, out=out)
    assert _rel(out, A.float() @ B.float().t()) < 5e-3 and torch.isfinite(out.float()).all()


def test_gemm_grouped_layouts_and_epilogues():
    from nestor_b200.ops import gemm as G
    torch.manual_seed(1)
    rows, E, d, h = 5000, 12, 640, 216
    off = _offsets(rows, E, empty=(0, 5))
    o = off.tolist()
    X = torch.randn(rows, d, device="cuda").to(BF)
    Wg, Wu = (torch.randn(E, d, h, device="cuda") * 0.05).to(BF), (torch.randn(E, d, h, device="cuda") * 0.05).to(BF)
    Wd = (torch.randn(E, h, d, device="cuda") * 0.05).to(BF)
    H = torch.full((rows, h), float("nan"), device="cuda", dtype=BF)
    Gt, Ut = torch.empty_like(H), torch.empty_like(H)
    G.gemm_rows(X, Wg, B2=Wu, offsets=off, groups=E, b_mn=True, out=H, epilogue=G.SWIGLU, extra_out=(Gt, Ut))
    g = torch.cat([X[o[e]:o[e + 1]].float() @ Wg[e].float() for e in range(E)])
    u = torch.cat([X[o[e]:o[e + 1]].float() @ Wu[e].float() for e in range(E)])
    assert _rel(Gt, g) < 5e-3 and _rel(Ut, u) < 5e-3
    assert _rel(H, torch.nn.functional.silu(g.to(BF)).float() * u.to(BF).float()) < 1e-2
    Y = torch.full((rows, d), float("nan"), device="cuda", dtype=BF)
    G.gemm_rows(H, Wd, offsets=off, groups=E, b_mn=True, out=Y)                              # MN-major B
    assert _rel(Y, torch.cat([H[o[e]:o[e + 1]].float() @ Wd[e].float() for e in range(E)])) < 5e-3
    dG, dU = torch.randn(rows, h, device="cuda").to(BF), torch.randn(rows, h, device="cuda").to(BF)
    dX = G.gemm_rows(dG, Wg, A2=dU, B2=Wu, offsets=off, groups=E)                            # two reduction segments
    want = torch.cat([dG[o[e]:o[e + 1]].float() @ Wg[e].float().t() + dU[o[e]:o[e + 1]].float() @ Wu[e].float().t() for e in range(E)])
    assert _rel(dX, want) < 5e-3
    acc0 = torch.randn(E, d, h, device="cuda")
    acc = acc0.clone()
    G.gemm_reduce(X, dG, offsets=off, groups=E, out=acc)                                     # weight gradient, accumulate
    want = acc0 + torch.stack([X[o[e]:o[e + 1]].float().t() @ dG[o[e]:o[e + 1]].float() for e in range(E)])
    assert _rel(acc, want) < 1e-4
    st = torch.full((E, d, h), float("nan"), device="cuda")
    G.gemm_reduce(X, dG, offsets=off, groups=E, out=st, epilogue=G.STORE_F32)
    assert (st[0] == 0).all() and _rel(st, want - acc0) < 1e-4                               # empty group -> zeros
    small = torch.zeros(8, d, device="cuda")
    G.gemm_reduce(dG[:, :8].contiguous(), X, out=small)                                      # split reduction path
    assert _rel(small, dG[:, :8].float().t() @ X.float()) < 1e-4


@pytest.mark.parametrize("M,N,E", [(640, 216, 12), (200, 600, 8), (1000, 256, 3), (640, 128, 1)])
def test_gemm_reduce_on_cta_pairs_and_single_ctas(M, N, E):
    """Weight-gradient products: the CTA-pair kernel (256-row tiles, each CTA staging half of B) and the single-CTA
    kernel against the fp32 statement, with ragged groups (partial last k-block of every group), an empty group,
    M that is not a multiple of the tile and both output epilogues."""

    from nestor_b200.ops import gemm as G
    torch.manual_seed(3)
    rows = 3000
    off = _offsets(rows, E, empty=(1,)) if E > 2 else torch.tensor([0, rows] if E == 1 else [0, 1111, rows], dtype=torch.int32, device="cuda")
    o = off.tolist()
    A = G.rows_buffer(rows, M, BF, "cuda"); A.copy_(torch.randn(rows, M, device="cuda"))
    B = G.rows_buffer(rows, N, BF, "cuda"); B.copy_(torch.randn(rows, N, device="cuda"))
    want = torch.stack([A[o[e]:o[e + 1]].float().t() @ B[o[e]:o[e + 1]].float() for e in range(E)])
    for pair in (True, False):
        st = torch.full((E, M, N), float("nan"), device="cuda")
        G.gemm_reduce(A, B, offsets=off, groups=E, out=st, epilogue=G.STORE_F32, pair=pair)
        assert torch.isfinite(st).all() and _rel(st, want) < 1e-4, (pair, "store")
        acc0 = torch.randn(E, M, N, device="cuda")
        acc = acc0.clone()
        G.gemm_reduce(A, B, offsets=off, groups=E, out=acc, alpha=0.5, pair=pair)
        assert _rel(acc, acc0 + 0.5 * want) < 1e-4, (pair, "accumulate")


def test_gemm_stats_epilogue_gives_logsumexp():
    from nestor_b200.ops import gemm as G
    torch.manual_seed(2)
    T, V, d = 700, 10023, 640
    ld = -(-V // 8) * 8
    h, W = torch.randn(T, d, device="cuda").to(BF), (torch.randn(V, d, device="cuda") * 0.1).to(BF)
    nt = -(-ld // 256)
    logits = torch.empty(T, ld, device="cuda", dtype=BF)
    part = torch.zeros(T, nt * G.STATS_PARTS, 2, device="cuda")
    G.gemm_rows(h, W, out=logits, epilogue=G.STORE_BF16_STATS, alpha=0.125, bn=256, extra_out=(part,), n=ld, n_valid=V)
    m = part[..., 0].max(1).values
    lse = m + torch.log((part[..., 1] * torch.exp(part[..., 0] - m[:, None])).sum(1))
    assert _rel(lse, torch.logsumexp(logits[:, :V].float(), 1)) < 1e-4
    assert torch.isinf(logits[:, V:].float()).all()


@pytest.mark.parametrize("lazy", [False, True])
@pytest.mark.parametrize("H,hd,lens", [(5, 40, [300, 1, 129, 128, 0, 700]), (2, 80, [600, 257]), (3, 64, [512, 64]), (4, 32, [900])])
def test_flash_forward_backward(H, hd, lens, lazy, monkeypatch):
    from nestor_b200.ops import flash as F
    monkeypatch.setattr(F, "LAZY_RESCALE", lazy)     # output accumulator in TMEM with rare rescales / in registers
    torch.manual_seed(3)
    rows, inner = sum(lens), H * hd
    qkv = torch.randn(rows, 3 * inner, device="cuda").to(BF)
    seg = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
    q, k, v = qkv[:, :inner], qkv[:, inner:2 * inner], qkv[:, 2 * inner:]
    out = torch.full((rows, inner), float("nan"), device="cuda", dtype=BF)
    o, lse = F.flash_fwd(q, k, v, seg, H, hd, 1.0 / hd, out=out)
    qr = qkv.float().clone().requires_grad_(True)
    ref = torch.zeros(rows, H, hd, device="cuda")
    ref_lse = torch.zeros(rows, H, device="cuda")
    s = seg.tolist()
    for a, b in zip(s[:-1], s[1:]):
        if b <= a:
            continue
        qq, kk, vv = (qr[a:b, i * inner:(i + 1) * inner].reshape(b - a, H, hd).transpose(0, 1) for i in range(3))
        sc = (qq @ kk.transpose(1, 2)) / hd
        sc = sc.masked_fill(~torch.ones(b - a, b - a, dtype=torch.bool, device="cuda").tril(), float("-inf"))
        ref_lse[a:b] = (torch.logsumexp(sc, -1) / math.log(2)).transpose(0, 1).detach()
        ref = ref.index_put((torch.arange(a, b, device="cuda"),), (torch.softmax(sc, -1) @ vv).transpose(0, 1))
    assert _rel(o, ref.reshape(rows, inner)) < 1e-2 and (lse - ref_lse).abs().max() < 2e-2
    do = torch.randn(rows, inner, device="cuda").to(BF)
    dqkv = torch.full((rows, 3 * inner), float("nan"), device="cuda", dtype=BF)
    F.flash_bwd(q, k, v, o, do, lse, seg, H, hd, 1.0 / hd, dqkv=dqkv)
    (ref.reshape(rows, inner) * do.float()).sum().backward()
    for i in range(3):
        sl = slice(i * inner, (i + 1) * inner)
        assert _rel(dqkv[:, sl], qr.grad[:, sl]) < 2e-2
    assert torch.isfinite(dqkv.float()).all()


def test_flash_forward_with_softmax_warps_at_different_speeds_is_exact_and_repeatable():
    """The four softmax warps of a q tile run independently and may be a kv tile apart. Here one quarter of every q
    tile has row maxima that grow with every kv tile (those warps rescale the accumulator each time, the others
    never do), which pulls the warps apart; the output must still match the fp32 statement and be bit-identical
    over repeated launches (a product issued before a slow warp has written its probabilities reads stale rows)."""

    from nestor_b200.ops import flash as F
    torch.manual_seed(11)
    H, hd, L, nseg = 3, 40, 1536, 6
    rows, inner = L * nseg, H * hd
    q = torch.randn(rows, H, hd, device="cuda") * 0.5
    k = torch.randn(rows, H, hd, device="cuda") * 0.5
    v = torch.randn(rows, H, hd, device="cuda")
    pos = torch.arange(rows, device="cuda") % L
    slow = ((torch.arange(rows, device="cuda") % 128) >= 96).float()[:, None, None]     # the last warp of each q tile
    q = q + slow * 3.0                                     # its scores follow k[..., 0] ...
    q[..., 0] = q[..., 0] * (1 - slow[..., 0]) + slow[..., 0] * 40.0
    k[..., 0] = (pos.float() / L)[:, None] * 12.0          # ... which grows along the sequence: a new maximum per tile
    qkv = torch.cat([q.reshape(rows, inner), k.reshape(rows, inner), v.reshape(rows, inner)], 1).to(BF)
    seg = torch.arange(0, rows + 1, L, dtype=torch.int32, device="cuda")
    qq, kk, vv = qkv[:, :inner], qkv[:, inner:2 * inner], qkv[:, 2 * inner:]
    first, _ = F.flash_fwd(qq, kk, vv, seg, H, hd, 1.0 / hd)
    first = first.clone()
    want = torch.empty(rows, H, hd, device="cuda")
    for a in range(0, rows, L):
        q3, k3, v3 = (t[a:a + L].float().reshape(L, H, hd).transpose(0, 1) for t in (qq, kk, vv))
        sc = (q3 @ k3.transpose(1, 2)) / hd
        sc = sc.masked_fill(~torch.ones(L, L, dtype=torch.bool, device="cuda").tril(), float("-inf"))
        want[a:a + L] = (torch.softmax(sc, -1) @ v3).transpose(0, 1)
    assert _rel(first, want.reshape(rows, inner)) < 1e-2
    junk = torch.randn(4096, 4096, device="cuda")
    for i in range(25):
        if i % 5 == 0:
            junk = junk @ junk.t() * 1e-4          # other kernels in between: the attention kernel starts from a cold cache
        again, _ = F.flash_fwd(qq, kk, vv, seg, H, hd, 1.0 / hd)
        assert torch.equal(again, first), i


@pytest.mark.parametrize("nsrc,d", [(3, 640), (9, 640), (47, 640), (5, 256), (4, 1280)])
def test_depth_read_norm(nsrc, d):
    from nestor_b200.ops import cuda as K, reference as R
    torch.manual_seed(4)
    T = 555
    srcs = [(torch.randn(T, d, device="cuda") * (0.1 + i)).requires_grad_(True) for i in range(nsrc)]
    q = (torch.randn(d, device="cuda") * 0.3).requires_grad_(True)
    gn = (torch.rand(50, device="cuda") + 0.5).requires_grad_(True)
    gm = (torch.rand(d, device="cuda") + 0.5).requires_grad_(True)
    out = K.depth_read_norm(srcs, q, gn, gm, 1e-6, 1e-5, BF)
    gg = torch.randn(T, d, device="cuda").to(BF).float()
    (out.float() * gg).sum().backward()
    s2 = [s.detach().clone().requires_grad_(True) for s in srcs]
    q2, gn2, gm2 = (t.detach().clone().requires_grad_(True) for t in (q, gn, gm))
    (R.depth_read_norm(s2, q2, gn2, gm2, 1e-6, 1e-5, torch.float32) * gg).sum().backward()
    assert _rel(q.grad, q2.grad) < 1e-4 and _rel(gn.grad, gn2.grad) < 1e-4 and _rel(gm.grad, gm2.grad) < 1e-4
    assert _rel(srcs[0].grad, s2[0].grad) < 1e-4 and _rel(srcs[-1].grad, s2[-1].grad) < 1e-4


def test_fused_ops_match_oracle_forward_and_backward():
    from nestor_b200.ops import cuda as K, reference as R
    torch.manual_seed(5)
    d = 640
    # expert bank
    T, E, h, slots, group = 1500, 16, 216, 4, 2
    x = torch.randn(T, d, device="cuda", requires_grad=True)
    ids, wts = torch.randint(0, E, (T, slots), device="cuda"), torch.rand(T, slots, device="cuda", requires_grad=True)
    ws = [(torch.randn(*s, device="cuda") * 0.04).to(BF).requires_grad_(True) for s in ((E, d, h), (E, d, h), (E, h, d))]
    plan = R.build_expert_plan(ids, E)
    out = K.expert_bank(x, plan, wts, *ws, BF, group)
    gg = torch.randn_like(out)
    (out * gg).sum().backward()
    x2, wts2 = x.detach().clone().requires_grad_(True), wts.detach().clone().requires_grad_(True)
    ws2 = [w.detach().clone().requires_grad_(True) for w in ws]
    (R.expert_bank(x2, plan, wts2, *ws2, BF, group) * gg).sum().backward()
    assert _rel(x.grad, x2.grad) < 2e-2 and _rel(wts.grad, wts2.grad) < 2e-2
    assert all(_rel(a.grad, b.grad) < 2e-2 for a, b in zip(ws, ws2))
    # column attention
    B, S, Gc, k, H, hd = 2, 384, 8, 3, 5, 40
    T, inner = B * S, H * hd
    n = torch.randn(T, d, device="cuda", requires_grad=True)
    idx = torch.randn(B, S, Gc, device="cuda").topk(k, -1).indices
    gates = torch.rand(T, k, device="cuda", requires_grad=True)
    plan = R.build_column_plan(idx, Gc)
    wqkv = (torch.randn(Gc, 3 * inner, d, device="cuda") * 0.04).to(BF).requires_grad_(True)
    wo = (torch.randn(Gc, d, inner, device="cuda") * 0.04).to(BF).requires_grad_(True)
    out = K.column_attention(n, plan, gates, wqkv, wo, H, hd, 1e4, BF)
    gg = torch.randn_like(out)
    (out * gg).sum().backward()
    n2, g2, wq2, wo2 = (t.detach().clone().requires_grad_(True) for t in (n, gates, wqkv, wo))
    out2 = R.column_attention(n2, plan, g2, wq2, wo2, H, hd, 1e4, BF)
    (out2 * gg).sum().backward()
    assert _rel(out, out2) < 1e-2
    for a, b in ((n, n2), (gates, g2), (wqkv, wq2), (wo, wo2)):
        assert _rel(a.grad, b.grad) < 2e-2
    # head + cross-entropy (vocabulary not a multiple of 8)
    T, V = 900, 100263
    hdn = torch.randn(T, d, device="cuda").to(BF).requires_grad_(True)
    W = (torch.randn(V, d, device="cuda") * 0.1).to(BF).requires_grad_(True)
    tg = torch.randint(0, V, (T,), device="cuda")
    tg[::7] = -100
    ls, cnt = K.lm_head_ce(hdn, W, tg, 0.125, BF, chunk_rows=512)
    (ls / cnt).backward()
    h2, W2 = hdn.detach().clone().requires_grad_(True), W.detach().clone().requires_grad_(True)
    ls2, cnt2 = R.lm_head_ce(h2, W2, tg, 0.125, BF, chunk_rows=512)
    (ls2 / cnt2).backward()
    assert int(cnt) == int(cnt2) and abs(float(ls) - float(ls2)) / float(ls2) < 2e-3
    assert _rel(hdn.grad, h2.grad) < 2e-2 and _rel(W.grad, W2.grad) < 2e-2
    # stream bookkeeping
    T, k = 300, 3
    attn, priv = torch.randn(T, k, d, device="cuda", requires_grad=True), torch.randn(T, k, d, device="cuda", requires_grad=True)
    pub = torch.randn(T, d, device="cuda", requires_grad=True)
    path = torch.softmax(torch.randn(T, 2, device="cuda"), -1).requires_grad_(True)
    st, rn = torch.randn(T, k, d, device="cuda", requires_grad=True), torch.randn(T, d, device="cuda", requires_grad=True)
    s1, r1 = K.layer_combine(attn, priv, pub, path, st, rn, BF)
    dev, agg = K.block_exit(s1)
    mid = K.mid_source(r1, attn)
    w = [torch.randn_like(t) for t in (dev, agg, mid)]
    ((dev * w[0]).sum() + (agg * w[1]).sum() + (mid * w[2]).sum()).backward()
    leaves = (attn, priv, pub, path, st, rn)
    clones = [t.detach().clone().requires_grad_(True) for t in leaves]
    s2, r2 = R.layer_combine(*clones[:4], clones[4], clones[5], BF)
    dev2, agg2 = R.block_exit(s2)
    mid2 = R.mid_source(r2, clones[0])
    ((dev2 * w[0]).sum() + (agg2 * w[1]).sum() + (mid2 * w[2]).sum()).backward()
    assert _rel(s1, s2) < 1e-5 and _rel(dev, dev2) < 1e-5
    for a, b in zip(leaves, clones):
        assert _rel(a.grad, b.grad) < 2e-2, a.shape


@pytest.mark.parametrize("family,variant", [
    ("nestor", {}), ("moe", {}), ("dense", {}),
    ("moe", {"router_num_dense_shared_experts": 1}),          # an always-on expert beside the routed bank
    ("nestor", {"block_expert_pool_public_experts": 0}),      # private-only pools: no public path, no path gate
    # merged blocks, a merged leading layer in the two-layer blocks, mass-conserving gains, per-source head queries
    ("nestor", {"_layers": (2, 1, 1, 1, 1, 1, 2), "block_column_blocks": [1, 2, 6], "block_column_trailing_layers": 1,
                "block_column_mass_lambda": 0.3, "block_column_gain_init": 1.0,
                "block_column_head_query_per_source": True}),
    # column-resolved sublayer reads (strided live columns beside every earlier export)
    ("nestor", {"_layers": (2, 1, 1, 1, 1, 1, 2), "block_column_head_only": False, "block_column_gain_init": 0.25}),
    # multi-column blocks under the merged recurrence
    ("nestor", {"block_residual_mode": "attn_res_kimi", "block_column_head_only": False,
                "block_column_include_aggregate": False, "block_column_deviation_sources": False,
                "block_column_gain_init": 1.0}),
    # pointwise experts in banks whose size changes with depth
    ("moe", {"block_mlp_activations": "gelu", "router_num_dense_shared_experts": 1,
             "block_layer_num_experts": [[5], [9], [4], [12]], "router_num_shared_experts": [3, 4, 4, 0]}),
    # within-block history attention joined by the between-block mixture
    ("moe", {"residual_mode": "attn_res", "block_residual_mode": "attn_res"}),
    # banks with column-specific experts in multi-column blocks (merged recurrence)
    ("moe", {"num_groups": [4] * 4, "num_groups_per_token": [2, 2, 1, 3], "block_num_heads": [2] * 4,
             "router_num_experts_per_group": [6, 5, 6, 4], "router_num_shared_experts": [2, 0, 3, 4],
             "router_num_experts_per_group_per_token": [3, 2, 3, 2], "router_score_mlp_hidden_dims": [[16]] * 4,
             "router_noise_mlp_hidden_dims": [[16]] * 4, "attention_token_dispatch": True}),
    # bidirectional attention (the two attention ops leave the kernels, everything else stays)
    ("nestor", {"causal": False}),
])
def test_whole_model_kernels_vs_oracle_with_pinned_routing(family, variant, tiny_scale, monkeypatch):
    import dataclasses as dc
    from nestor_b200 import ops
    from nestor_b200.models import Model
    from nestor_b200.parallel.arena import ParamArena
    from nestor_b200.train.losses import CausalLMLoss
    variant = dict(variant)
    monkeypatch.setitem(tiny_scale.SCALES, "tiny", tiny_scale.Scale("tiny", 256, 4, 16, 1024, 10, 2, 1024))
    monkeypatch.setitem(tiny_scale.NESTOR_LAYERS, "tiny", variant.pop("_layers", (1,) * 7))
    monkeypatch.setenv("DCLM_BLOCK_SIZE", "512")
    torch.manual_seed(1)
    cfg = tiny_scale.build_experiment(family, "tiny").jobs[0].model
    cfg = dc.replace(cfg, backbone_config=dc.replace(cfg.backbone_config, **variant))
    m = Model.from_config(cfg).cuda().eval()
    with torch.no_grad():
        for name, p in m.named_parameters():
            if "query" in name:
                # (history-attention logits have no 1/sqrt(d) temperature: keep that softmax well conditioned)
                p.normal_(0, 0.1 if variant.get("residual_mode") == "attn_res" else 0.3)
    m.compute_dtype, m.fused_head = BF, True
    arena = ParamArena(m, compute_dtype=BF, device=torch.device("cuda"))
    ids = torch.randint(0, 100263, (2, 512), device="cuda")
    tape, res = ops.RoutingTape(), {}
    try:
        for mode in ("kernels", "oracle"):
            monkeypatch.setattr(ops, "_FORCE_REF", mode == "oracle")
            ops.set_routing_tape(tape, "record" if mode == "kernels" else "replay")
            arena.zero_grad()
            out = m(ids)
            loss = CausalLMLoss()(out.pred, ids, out.aux).total
            loss.backward()
            res[mode] = (float(loss), arena.grad.clone())
    finally:
        ops.set_routing_tape(None)
    assert abs(res["kernels"][0] - res["oracle"][0]) < 2e-3
    assert _rel(res["kernels"][1], res["oracle"][1]) < 5e-2


def test_bounded_wait_reports_timeout_and_context_survives():
    from nestor_b200.parallel.symm import wait_timeout_probe
    code = wait_timeout_probe(torch.device("cuda"), budget=2000)
    assert code == 5                                   # kTimeoutPeer
    assert float(torch.ones(4, device="cuda").sum()) == 4.0


def test_graphed_step_matches_eager_and_smoke(monkeypatch):
    import __graft_entry__ as entry
    entry.smoke()
    from nestor_b200.experiments.tiny import nestor_tiny
    from nestor_b200.models import Model
    from nestor_b200.train.trainer import Trainer
    losses = {}
    for flag in ("0", "1"):
        monkeypatch.setenv("NESTOR_B200_CUDA_GRAPH", flag)
        torch.manual_seed(0)
        job = nestor_tiny().jobs[0]
        tr = Trainer(job, Model.from_config(job.model), [], device=torch.device("cuda"))
        tr.model.eval()                                 # deterministic routing (no exploration noise)
        tr.model.training = True
        for blk in tr.model.backbone.blocks:
            blk.freeze_routing_noise = True
        vals = []
        for step in range(5):
            g = torch.Generator().manual_seed(step)
            ids = torch.randint(0, 100277, (2, 256), generator=g)
            loss, counts = tr.train_step((ids, ids))
            tr.update_weights(counts)
            vals.append(float(loss.total))
        losses[flag] = vals
        assert (tr._graph is not None) == (flag == "1")
    assert all(abs(a - b) < 5e-3 for a, b in zip(losses["0"], losses["1"])), losses


def test_route_and_plan_kernels_match_oracle():
    from nestor_b200 import ops
    from nestor_b200.ops import cuda as K, reference as R
    torch.manual_seed(5)
    T, P, Gc, Q, kc, kq = 3000, 12, 8, 8, 3, 2
    width = P + Gc * Q + 2
    base = torch.randn(T, width, device="cuda").to(BF)
    bias_p, bias_q = torch.randn(P, device="cuda") * 0.1, torch.randn(Gc, Q, device="cuda") * 0.1
    cols = torch.rand(T, Gc, device="cuda").topk(kc, dim=-1).indices
    cg = torch.rand(T, kc, device="cuda") + 0.1
    tape = ops.RoutingTape()

    def run(mod, mode):
        s = base.clone().requires_grad_()
        g = cg.clone().requires_grad_()
        ops.set_routing_tape(tape, mode)
        pub_idx, pub_gate = mod.route_topk(s[:, :P], bias_p, 4, "renorm")
        out = {}
        for gm in ("renorm", "switch"):
            out[gm] = mod.route_selected(s[:, P:P + Gc * Q].reshape(T, Gc, Q), bias_q, cols, g, kq, gm, BF)
        ops.set_routing_tape(None)
        loss = (pub_gate * torch.arange(1, 5, device="cuda")).sum()
        for gm, (ids, w, _) in out.items():
            loss = loss + (w.float() * torch.linspace(0.5, 1.5, kc * kq, device="cuda")).sum()
        loss.backward()
        return pub_idx, pub_gate, out, s.grad, g.grad

    a = run(K, "record")
    b = run(R, "replay")
    assert torch.equal(a[0].long(), b[0].long()) and _rel(a[1], b[1]) < 1e-5
    for gm in ("renorm", "switch"):
        assert torch.equal(a[2][gm][0].long(), b[2][gm][0].long())
        assert _rel(a[2][gm][1], b[2][gm][1]) < 1e-2
    assert _rel(a[3], b[3]) < 2e-2 and _rel(a[4], b[4]) < 2e-2
    # free selection: the chosen entries carry the k largest biased scores
    idx, _ = K.route_topk(base[:, :P], bias_p, 4, "renorm")
    biased = base[:, :P].float() + bias_p
    assert torch.allclose(biased.gather(1, idx.long()).sort(1).values, biased.topk(4, dim=1).values.sort(1).values)
    ids = torch.randint(0, 24, (5000, 3), device="cuda")
    pa, pb = K.build_expert_plan(ids, 24), R.build_expert_plan(ids, 24)
    assert torch.equal(pa.order, pb.order) and torch.equal(pa.inv, pb.inv) and torch.equal(pa.offsets, pb.offsets)


def test_multi_tensor_optimizer_matches_foreach(monkeypatch):
    from nestor_b200.train import optim as O
    torch.manual_seed(7)

    def make():
        torch.manual_seed(7)
        mats = [torch.nn.Parameter(torch.randn(64, 96, device="cuda")), torch.nn.Parameter(torch.randn(3, 48, 32, device="cuda"))]
        vecs = [torch.nn.Parameter(torch.randn(1000, device="cuda")), torch.nn.Parameter(torch.randn(70000, device="cuda"))]
        groups = [dict(params=mats, method="muon", lr=0.02, weight_decay=0.1, momentum=0.95, nesterov=True, ns_steps=5),
                  dict(params=vecs, method="adamw", lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)]
        return mats + vecs, O.MuonAdamW(groups)

    pa, oa = make()
    pb, ob = make()
    for step in range(3):
        for x, y in zip(pa, pb):
            g = torch.randn_like(x)
            x.grad, y.grad = g.clone(), g.clone()
        oa.step()
        with monkeypatch.context() as m:
            m.setattr(O, "_fused", lambda *a: False)
            ob.step()
    for x, y in zip(pa, pb):
        assert _rel(x, y) < 1e-5


def test_column_plan_kernel_matches_oracle():
    from nestor_b200.ops import cuda as K, reference as R
    torch.manual_seed(11)
    for (B, S, Gc, k, with_pos) in [(4, 512, 8, 3, False), (2, 300, 8, 6, True), (16, 64, 8, 8, False)]:
        idx = torch.rand(B, S, Gc, device="cuda").topk(k, dim=-1).indices
        pos = torch.randint(0, 4 * S, (B, S), device="cuda") if with_pos else None
        a, b = K.build_column_plan(idx, Gc, pos), R.build_column_plan(idx, Gc, pos)
        for f in ("row_of_slot", "tok_of_row", "slot_of_row", "pos_of_row", "seg_start", "col_start", "idx"):
            assert torch.equal(getattr(a, f).long(), getattr(b, f).long()), f


def test_flash_lazy_rescale_follows_growing_maxima(monkeypatch):
    """Scores that keep growing along the sequence force the TMEM-resident accumulator to be rescaled many times."""

    from nestor_b200.ops import flash as F
    monkeypatch.setattr(F, "LAZY_RESCALE", True)
    torch.manual_seed(9)
    H, hd, n = 2, 40, 700
    inner = H * hd
    q = (torch.randn(n, inner, device="cuda") * 6).to(BF)
    k = (torch.randn(n, inner, device="cuda") * (1 + torch.arange(n, device="cuda")[:, None] / 20.0)).to(BF)
    v = torch.randn(n, inner, device="cuda").to(BF)
    seg = torch.tensor([0, n], dtype=torch.int32, device="cuda")
    o, lse = F.flash_fwd(q, k, v, seg, H, hd, 1.0 / hd)
    qq, kk, vv = (t.float().reshape(n, H, hd).transpose(0, 1) for t in (q, k, v))
    sc = (qq @ kk.transpose(1, 2)) / hd
    sc = sc.masked_fill(~torch.ones(n, n, dtype=torch.bool, device="cuda").tril(), float("-inf"))
    ref = (torch.softmax(sc, -1) @ vv).transpose(0, 1).reshape(n, inner)
    assert (sc.amax(-1).diff(dim=-1) > 0).float().mean() > 0.2        # the maxima do move
    assert _rel(o, ref) < 1e-2
    assert (lse - (torch.logsumexp(sc, -1) / math.log(2)).transpose(0, 1)).abs().max() < 5e-2


@pytest.mark.parametrize("d,H,hd,Gc,k", [(480, 5, 30, 8, 3), (960, 3, 60, 8, 5), (480, 16, 30, 1, 1)])
def test_attention_with_head_dims_that_are_not_multiples_of_eight(d, H, hd, Gc, k):
    """The 100m (head_dim 30) and 500m (head_dim 60) scales: heads are re-pitched around the attention kernels."""

    from nestor_b200.ops import cuda as K, reference as R
    torch.manual_seed(6)
    B, S = 2, 320
    T, inner = B * S, H * hd
    n = torch.randn(T, d, device="cuda", requires_grad=True)
    wqkv = (torch.randn(Gc, 3 * inner, d, device="cuda") * 0.04).to(BF).requires_grad_(True)
    wo = (torch.randn(Gc, d, inner, device="cuda") * 0.04).to(BF).requires_grad_(True)
    gg = torch.randn(T, k, d, device="cuda")
    n2, wq2, wo2 = (t.detach().clone().requires_grad_(True) for t in (n, wqkv, wo))
    if Gc > 1:
        idx = torch.randn(B, S, Gc, device="cuda").topk(k, -1).indices
        gates = torch.rand(T, k, device="cuda", requires_grad=True)
        g2 = gates.detach().clone().requires_grad_(True)
        plan = R.build_column_plan(idx, Gc)
        out = K.column_attention(n, plan, gates, wqkv, wo, H, hd, 1e4, BF)
        out2 = R.column_attention(n2, plan, g2, wq2, wo2, H, hd, 1e4, BF)
        pairs = [(n, n2), (gates, g2), (wqkv, wq2), (wo, wo2)]
    else:
        out = K.dense_attention(n, B, S, wqkv, wo, H, hd, 1e4, BF).view(T, 1, d)
        out2 = R.dense_attention(n2, B, S, wq2, wo2, H, hd, 1e4, BF).view(T, 1, d)
        pairs = [(n, n2), (wqkv, wq2), (wo, wo2)]
    (out * gg).sum().backward()
    (out2 * gg).sum().backward()
    assert _rel(out, out2) < 1e-2
    for a, b in pairs:
        assert _rel(a.grad, b.grad) < 2e-2


@pytest.mark.parametrize("rows,world", [(9000, 4), (1500, 2)])
def test_gemm_with_fused_all_gather_of_rank_sharded_banks(rows, world):
    """Weights staged from their owners' arenas by the copy warps of the same launch (ranks emulated as local buffers).

    Every emulated arena holds valid values only for the groups its rank owns (NaN elsewhere, the local arena
    included), so a finite result equal to the ungathered product proves that each group came from its owner.
    """

    from nestor_b200.ops import gemm as G
    torch.manual_seed(5)
    E, d, h = 8, 640, 216
    per = E // world
    off = _offsets(rows, E, empty=(3,))
    X = torch.randn(rows, d, device="cuda").to(BF)
    Hh = torch.randn(rows, h, device="cuda").to(BF)
    Wg, Wu = (torch.randn(E, d, h, device="cuda") * 0.05).to(BF), (torch.randn(E, d, h, device="cuda") * 0.05).to(BF)
    Wd = (torch.randn(E, h, d, device="cuda") * 0.05).to(BF)
    # arena layout: [pad | gate | up | down(strided groups)]; the down bank sits at a group stride wider than a group
    n_gu, n_d, gap = E * d * h, h * d, 64
    o_g, o_u, o_d = 128, 128 + n_gu, 128 + 2 * n_gu
    total = o_d + E * (n_d + gap)
    arenas = []
    for r in range(world):
        a = torch.full((total,), float("nan"), device="cuda", dtype=BF)
        lo, hi = r * per, (r + 1) * per
        a[o_g : o_g + n_gu].view(E, d, h)[lo:hi] = Wg[lo:hi]
        a[o_u : o_u + n_gu].view(E, d, h)[lo:hi] = Wu[lo:hi]
        torch.as_strided(a, (E, h, d), (n_d + gap, d, 1), o_d)[lo:hi] = Wd[lo:hi]
        arenas.append(a)
    local = arenas[0]
    vg, vu = local[o_g : o_g + n_gu].view(E, d, h), local[o_u : o_u + n_gu].view(E, d, h)
    vd = torch.as_strided(local, (E, h, d), (n_d + gap, d, 1), o_d)
    stage = torch.full((2 * n_gu,), float("nan"), device="cuda", dtype=BF)
    flags = torch.zeros(257, dtype=torch.int32, device="cuda")
    spec = G.Gather(src=[a.data_ptr() for a in arenas], arena_ptr=local.data_ptr(), stage=stage, flags=flags,
                    groups_per_rank=per)

    def run(gather, wg, wu, wd):
        H = torch.full((rows, h), float("nan"), device="cuda", dtype=BF)
        Gt, Ut = torch.empty_like(H), torch.empty_like(H)
        G.gemm_rows(X, wg, B2=wu, offsets=off, groups=E, b_mn=True, out=H, epilogue=G.SWIGLU, extra_out=(Gt, Ut),
                    gather=gather)
        Y = G.gemm_rows(Hh, wd, offsets=off, groups=E, b_mn=True, gather=gather)          # down: MN-major B
        dH = G.gemm_rows(X, wd, offsets=off, groups=E, gather=gather)                     # K-major B [E, h, d]
        dX = G.gemm_rows(Hh, wg, A2=Hh, B2=wu, offsets=off, groups=E, gather=gather)      # two segments
        return H, Gt, Ut, Y, dH, dX

    import dataclasses
    want = run(None, Wg, Wu, Wd)
    # twice per ring shape (the counters must come back to zero between launches); the second shape has four
    # lanes of the copy warp copying independently
    for sp in (spec, spec, dataclasses.replace(spec, chunk=4096, nbuf=2, lanes=4), dataclasses.replace(spec, nbuf=2, lanes=4)):
        stage.fill_(float("nan"))
        got = run(sp, vg, vu, vd)
        torch.cuda.synchronize()
        assert int(flags.abs().sum().item()) == 0
        for w, g in zip(want, got):
            assert torch.isfinite(g.float()).all()
            assert torch.equal(w, g)


@pytest.mark.parametrize("shape", [(3, 200, 640), (2, 640, 200), (5, 216, 640), (4, 640, 216), (1, 128, 640), (2, 640, 640),
                                   (3, 80, 640), (2, 90, 480), (1, 640, 856), (300, 120, 640)])
def test_newton_schulz_matches_oracle(shape):
    """The tcgen05 Newton-Schulz against the fp32-input PyTorch statement, and orthogonality of the result.

    The iteration is run in bf16 on both sides with different rounding points, so the two results are compared
    loosely (bf16 noise amplified over five iterations); the singular values, which is what the optimizer relies on,
    must land in the same band as the oracle's.
    """

    from nestor_b200.ops import cuda as K, reference as R
    torch.manual_seed(sum(shape))
    g = torch.randn(*shape, device="cuda")
    got = K.newton_schulz(g, 5)
    want = R.newton_schulz(g, 5)
    assert got.shape == want.shape and got.dtype == g.dtype and torch.isfinite(got).all()
    assert _rel(got, want) < 0.08, _rel(got, want)
    sv_got = torch.linalg.svdvals(got[0].float())
    sv_want = torch.linalg.svdvals(want[0].float())
    assert sv_got.max() < max(1.3, 1.05 * float(sv_want.max())) and sv_got.min() > min(0.3, 0.9 * float(sv_want.min()))
    # 2-D input and bf16 output
    one = K.newton_schulz(g[0], 5, out_dtype=BF)
    assert one.dtype == BF and one.shape == g[0].shape and _rel(one, got[0]) < 1e-2


def test_dispatch_refuses_cuda_tensor_without_kernel_body():
    from nestor_b200 import ops
    op = ops._dispatch("rope_tables") if hasattr(ops._ref, "rope_tables") else None
    x = torch.ones(4, device="cuda")
    if op is not None:
        with pytest.raises(RuntimeError, match="no sm_100a kernel body"):
            op(x)
    with ops.oracle_ops():
        assert not ops.use_kernels(x)
    assert ops.use_kernels(x)


def test_shape_beyond_a_kernel_limit_warns_counts_and_raises_when_strict(monkeypatch):
    """k = 9 is past the routing kernel's k <= 8: the call runs the PyTorch statement, says so once, is counted, and
    is an error under NESTOR_B200_STRICT=1."""

    from nestor_b200 import ops
    from nestor_b200.ops import reference as R
    scores = torch.randn(64, 32, device="cuda")
    bias = torch.zeros(32, device="cuda")
    before = ops.cuda_ops().oracle_path_report().get("route_topk", 0)
    ops.cuda_ops()._oracle_calls.pop("route_topk", None)
    with pytest.warns(RuntimeWarning, match="k <= 8"):
        idx, gates = ops.cuda_ops().route_topk(scores, bias, 9, "renorm")
    want_idx, want_gates = R.route_topk(scores, bias, 9, "renorm")
    assert torch.equal(idx, want_idx) and torch.allclose(gates, want_gates)
    assert ops.oracle_path_report()["route_topk"] == 1
    ops.cuda_ops()._oracle_calls["route_topk"] += before
    monkeypatch.setenv("NESTOR_B200_STRICT", "1")
    with pytest.raises(RuntimeError, match="no body for this shape"):
        ops.cuda_ops().route_topk(scores, bias, 9, "renorm")


def _poison_allocator(gib: float = 1.5):
    """Fill the caching allocator's free blocks with inf / NaN: memory a later ``torch.empty`` hands out is dirty, so
    any row or column a kernel leaves unwritten shows up in its output (the reference's dirty-allocator discipline,
    ``tests/test_triton_packed_attn.py:209-270``)."""

    sizes = [1 << 20, 4 << 20, 16 << 20, 64 << 20, 256 << 20]
    blocks = []
    budget = int(gib * (1 << 30))
    for i, sz in enumerate(sizes * 3):
        if budget < sz:
            break
        t = torch.empty(sz // 4, device="cuda")
        t.fill_(float("inf") if i % 2 else float("nan"))
        blocks.append(t)
        budget -= sz
    torch.cuda.synchronize()
    del blocks                      # freed blocks stay in the allocator's pool, poisoned


@pytest.mark.parametrize("shape", [(2, 96, 8, 3, 2, 40), (1, 200, 8, 8, 2, 40), (3, 64, 4, 2, 3, 30)])
def test_dirty_allocator_column_attention_and_expert_bank(shape):
    """Column attention and a routed expert bank on poisoned memory: outputs and gradients stay finite and equal the
    clean-memory run bit for bit (every buffer element that is read was written first)."""

    from nestor_b200.ops import cuda as K
    B, S, G, k, heads, hd = shape
    d, T = 64, B * S
    torch.manual_seed(5)
    n = torch.randn(T, d, device="cuda", requires_grad=True)
    scores = torch.randn(T, G, device="cuda")
    idx = scores.topk(k, dim=-1).indices.to(torch.int32)
    gates = torch.softmax(torch.randn(T, k, device="cuda"), -1).requires_grad_()
    inner = heads * hd
    wqkv = (torch.randn(G, 3 * inner, d, device="cuda") * 0.1).to(BF)
    wo = (torch.randn(G, d, inner, device="cuda") * 0.1).to(BF)
    E, h = 6, 48
    ids = torch.randint(0, E, (T, 2), device="cuda", dtype=torch.int32)
    ids[:, 0] = ids[:, 0].clamp_max(E - 2)                 # expert E-1 may stay empty in slot 0
    w = torch.rand(T, 2, device="cuda").to(BF)
    wu, wg = ((torch.randn(E, d, h, device="cuda") * 0.1).to(BF) for _ in range(2))
    wd = (torch.randn(E, h, d, device="cuda") * 0.1).to(BF)

    def run():
        plan = K.build_column_plan(idx.view(B, S, k), G) if G > 1 else None
        a = K.column_attention(n, plan, gates, wqkv, wo, heads, hd, 10000.0, BF)
        eplan = K.build_expert_plan(ids, E)
        e = K.expert_bank(n, eplan, w, wu, wg, wd, BF, group=2)
        ga, gg = torch.autograd.grad(a.sum() + e.sum(), (n, gates))
        return a.detach().clone(), e.detach().clone(), ga.clone(), gg.clone()

    clean = run()
    torch.cuda.synchronize()
    _poison_allocator()
    dirty = run()
    for c, x in zip(clean, dirty):
        assert torch.isfinite(x).all() and torch.equal(c, x)


def test_fastpath_check_prints_kernel_vs_oracle_difference(capsys, monkeypatch):
    """NESTOR_FASTPATH_CHECK=1: the first forwards are repeated on the PyTorch ops with the same routing."""

    import re
    monkeypatch.setenv("NESTOR_FASTPATH_CHECK", "1")
    monkeypatch.setenv("DCLM_DATA_PATH", "/tmp/unused.bin")
    from nestor_b200.experiments.tiny import nestor_tiny
    from nestor_b200.models import Model
    from nestor_b200.train.trainer import Trainer
    torch.manual_seed(0)
    job = nestor_tiny().jobs[0]
    m = Trainer(job, Model.from_config(job.model), [], device=torch.device("cuda")).model.eval()   # weights in the bf16 arena
    ids = torch.randint(0, 100277, (2, 128), device="cuda")
    with torch.no_grad():
        for _ in range(4):
            m(ids)
    out = capsys.readouterr().out
    diffs = [float(x) for x in re.findall(r"\[FASTPATH-CHECK\] max\|kernels - oracle\| = ([0-9.e+-]+)", out)]
    assert len(diffs) == 3 and max(diffs) < 0.25, out          # three checked forwards, bf16-level agreement


def test_gathering_gemm_wait_runs_out_and_context_survives():
    """The fused all-gather GEMM's B producer waits (bounded) for the copy warps to stage a group's weights. A group
    counter that can never reach its target makes that wait run out: the launch must come back with the peer-timeout
    status instead of hanging, leave the counters clean, and the next launch on the same context must be correct."""

    from nestor_b200.ops import _lib, gemm as G
    E, d, h, rows = 8, 128, 64, 2048
    torch.manual_seed(3)
    n = E * d * h
    arena = (torch.randn(n, device="cuda") * 0.05).to(BF)
    W = arena.view(E, d, h)
    X = torch.randn(rows, d, device="cuda").to(BF)
    off = (torch.arange(E + 1, dtype=torch.int32) * (rows // E)).cuda()
    stage = torch.empty(n, dtype=BF, device="cuda")
    flags = torch.zeros(257, dtype=torch.int32, device="cuda")
    spec = G.Gather(src=[arena.data_ptr()] * 8, arena_ptr=arena.data_ptr(), stage=stage, flags=flags, groups_per_rank=1,
                    wait_polls=20000)              # ~2 ms instead of the default half second
    want = G.gemm_rows(X, W, offsets=off, groups=E, b_mn=True)
    got = G.gemm_rows(X, W, offsets=off, groups=E, b_mn=True, gather=spec)
    torch.cuda.synchronize()
    _lib.check_status(torch.device("cuda"))
    assert torch.equal(got, want)
    flags[3] = -(1 << 20)                           # group 3 can never be reported complete
    G.gemm_rows(X, W, offsets=off, groups=E, b_mn=True, gather=spec)
    torch.cuda.synchronize()
    code = int(_lib.status_word(torch.device("cuda")).item())
    _lib.status_word(torch.device("cuda")).zero_()
    assert code == 5, code                          # kTimeoutPeer
    assert int(flags.abs().sum()) == 0              # the last CTA to leave cleared the counters
    again = G.gemm_rows(X, W, offsets=off, groups=E, b_mn=True, gather=spec)
    torch.cuda.synchronize()
    _lib.check_status(torch.device("cuda"))
    assert torch.equal(again, want)


def test_bounds_checking_build_records_a_bad_index_instead_of_reading_it():
    """The index-checking library build (NESTOR_B200_BOUNDS_CHECK=1): an out-of-range gather index is recorded in the
    status record and the row is skipped; valid rows are unaffected. Runs in a child process because a process loads
    one build of the library."""

    import os
    import subprocess
    import sys
    code = r"""
import torch
from nestor_b200.ops import cuda as K, _lib
assert _lib.lib().nb_bounds_check_enabled() == 1
src = torch.arange(6 * 64, dtype=torch.float32, device="cuda").view(6, 64)
idx = torch.tensor([0, 5, 17, 3], dtype=torch.int32, device="cuda")     # 17 is past the 6 source rows
assert K.bounds_check_report() is None
out = K.gather_rows(src, idx)
rep = K.bounds_check_report()
assert rep == {"code": 7, "kernel": "gather_rows", "index": 17, "row": 2}, rep
assert torch.equal(out[[0, 1, 3]].float(), src[[0, 5, 3]].bfloat16().float())
assert K.bounds_check_report() is None            # reading clears the record
y = torch.randn(8, 64, device="cuda").bfloat16()
bad = torch.tensor([1, 9], dtype=torch.int32, device="cuda")
o = K.combine_rows(y, bad, None, 1, 2)
assert K.bounds_check_report()["kernel"] == "combine_rows" and torch.equal(o[0], y[1].float()) and float(o[1].abs().sum()) == 0
print("BOUNDS_OK")
"""
    env = dict(os.environ, NESTOR_B200_BOUNDS_CHECK="1")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run([sys.executable, "-c", code], env=env, cwd=root, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and "BOUNDS_OK" in res.stdout, res.stdout + res.stderr


def test_fused_router_bias_update_matches_the_per_router_rule():
    """One kernel for every router: bias += rate * sign(mean(c) - c) on packed counts, against the PyTorch statement."""

    from nestor_b200.experiments.tiny import nestor_tiny
    from nestor_b200.models import Model
    from nestor_b200.models.nestor import RouterCounts, apply_bias_updates

    torch.manual_seed(5)
    m = Model.from_config(nestor_tiny().jobs[0].model).cuda()
    routers = {n: r for n, r in m.backbone.named_modules() if hasattr(r, "choice_bias") and getattr(r, "loss_free", False)}
    assert len(routers) >= 6
    counts = {n: torch.randint(0, 5, r.choice_bias.shape, device="cuda").float() for n, r in routers.items()}
    first = next(iter(counts))
    counts[first][:] = 3.0                                   # a router in perfect balance moves nothing
    want = {n: r.choice_bias.clone() + r.bias_rate * torch.sign(counts[n].mean() - counts[n]) for n, r in routers.items()}
    from nestor_b200 import ops
    before = ops.launch_count()
    apply_bias_updates(m.backbone, RouterCounts.pack(counts))
    assert ops.launch_count() == before + 1
    for n, r in routers.items():
        assert torch.allclose(r.choice_bias, want[n], atol=1e-7), n
    apply_bias_updates(m.backbone, RouterCounts.pack(counts))     # cached table, second application
    for n, r in routers.items():
        assert torch.allclose(r.choice_bias, want[n] + r.bias_rate * torch.sign(counts[n].mean() - counts[n]), atol=1e-7), n
