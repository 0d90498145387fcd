"""Plain-PyTorch statement of every hot op (the oracle, and the CPU execution path).

Each function here is the definition the sm_100a kernels in ``nestor_b200/csrc`` are
tested against: same inputs, same outputs, same rounding points (``cd`` is the compute
dtype — fp32 on CPU, bf16 on the GPU; accumulations, softmaxes and residual streams
are fp32). The data structures (``ColumnPlan``, ``ExpertPlan``) are the ones the
kernels consume, so the plan builders are shared between both paths.

Math references (reference repository paths): routing ``nestor/backbones/nestor.py:518-593``;
column attention ``:3206-3258`` / ``:6127-6267``; hybrid pool ``expert_pools.py:13-21``;
depth read ``attention_residual.py:488-718``; RMSNorm / RoPE ``scaling/blocks.py:346-438``;
chunked head+CE ``train/losses.py:228-272``; Newton–Schulz ``scaling/muon.py:83-151``.
"""

from __future__ import annotations

import dataclasses as dc
import math

import torch
import torch.nn.functional as F
from torch import Tensor

# ------------------------------------------------------------------------------ plans


@dc.dataclass
class ColumnPlan:
    """Packed layout of one block's column memberships (built once per block).

    Row ``r`` of the packed layout is one (token, slot) pair. Rows are ordered by
    (column, sequence, position), so the members of column ``c`` in sequence ``b`` form
    the contiguous segment ``seg_start[c*B+b] : seg_start[c*B+b+1]`` in token order, and
    causal attention inside a segment is plain lower-triangular. There is no alignment
    padding: ``rows == B*S*k`` exactly.

    Attributes:
        B, S, G, k: batch, sequence length, columns, columns per token.
        idx: ``[T, k]`` int32 column of each slot (router top-k order).
        row_of_slot: ``[T, k]`` int32 packed row holding slot ``j`` of token ``t``.
        tok_of_row: ``[rows]`` int32 flat token index of each packed row.
        slot_of_row: ``[rows]`` int32 slot index of each packed row.
        pos_of_row: ``[rows]`` int32 position (RoPE angle index) of each packed row.
        seg_start: ``[G*B + 1]`` int32 segment boundaries (column-major).
        col_start: ``[G + 1]`` int32 row range of each column (``seg_start[::B]``).
    """

    B: int
    S: int
    G: int
    k: int
    idx: Tensor
    row_of_slot: Tensor
    tok_of_row: Tensor
    slot_of_row: Tensor
    pos_of_row: Tensor
    seg_start: Tensor
    col_start: Tensor
    extra: dict = dc.field(default_factory=dict)

    @property
    def rows(self) -> int:
        return self.B * self.S * self.k


def build_column_plan(idx: Tensor, G: int, pos: Tensor | None = None) -> ColumnPlan:
    """Invert a ``[B, S, k]`` top-k column selection into the packed layout."""

    B, S, k = idx.shape
    dev = idx.device
    idx = idx.to(torch.int64)
    member = torch.zeros(B, S, G, dtype=torch.int32, device=dev)
    member.scatter_(2, idx, 1)
    # scan along the sequence with the scanned axis innermost (fast path of the scan kernels)
    rank = (member.transpose(1, 2).contiguous().cumsum(dim=-1, dtype=torch.int64) - 1).transpose(1, 2)  # [B,S,G]
    seg_len = member.sum(dim=1, dtype=torch.int64).transpose(0, 1).reshape(-1)   # [G*B], column-major
    seg_start = torch.zeros(G * B + 1, dtype=torch.int64, device=dev)
    seg_start[1:] = seg_len.cumsum(0)
    start_bc = seg_start[:-1].view(G, B).transpose(0, 1)              # [B,G]
    row_all = start_bc.unsqueeze(1) + rank                            # [B,S,G]
    row_of_slot = row_all.gather(2, idx).reshape(B * S, k)            # [T,k]
    rows = B * S * k
    tok = torch.arange(B * S, device=dev).unsqueeze(1).expand(-1, k)
    slot = torch.arange(k, device=dev).unsqueeze(0).expand(B * S, -1)
    tok_of_row = torch.empty(rows, dtype=torch.int64, device=dev)
    slot_of_row = torch.empty(rows, dtype=torch.int64, device=dev)
    tok_of_row[row_of_slot.reshape(-1)] = tok.reshape(-1)
    slot_of_row[row_of_slot.reshape(-1)] = slot.reshape(-1)
    if pos is None:
        pos_flat = torch.arange(S, device=dev).repeat(B)
    else:
        pos_flat = pos.reshape(-1).clamp_min(0).to(torch.int64)
    i32 = torch.int32
    return ColumnPlan(
        B=B, S=S, G=G, k=k,
        idx=idx.reshape(B * S, k).to(i32), row_of_slot=row_of_slot.to(i32),
        tok_of_row=tok_of_row.to(i32), slot_of_row=slot_of_row.to(i32),
        pos_of_row=pos_flat[tok_of_row].to(i32), seg_start=seg_start.to(i32),
        col_start=seg_start[:: B].contiguous().to(i32),
    )


@dc.dataclass
class ExpertPlan:
    """Rows of an expert bank grouped by expert (stable counting sort, no padding).

    Attributes:
        E: experts in the bank; n: rows (= tokens x slots).
        order: ``[n]`` int32, ``order[r]`` = flat (token*slots + slot) index feeding sorted row ``r``.
        inv: ``[n]`` int32 inverse permutation (sorted row of each flat slot).
        offsets: ``[E + 1]`` int32 row range of each expert.
        slots: slots per token.
    """

    E: int
    n: int
    slots: int
    order: Tensor
    inv: Tensor
    offsets: Tensor


def build_expert_plan(expert_ids: Tensor, E: int) -> ExpertPlan:
    """Group the flattened ``[T, slots]`` expert ids by expert, keeping slot order inside one."""

    T, slots = expert_ids.shape
    flat = expert_ids.reshape(-1).to(torch.int64)
    order = torch.sort(flat, stable=True).indices
    inv = torch.empty_like(order)
    inv[order] = torch.arange(order.numel(), device=order.device)
    counts = torch.zeros(E, dtype=torch.int64, device=flat.device).scatter_add_(0, flat, torch.ones_like(flat))
    offsets = torch.zeros(E + 1, dtype=torch.int64, device=flat.device)
    offsets[1:] = counts.cumsum(0)
    return ExpertPlan(E=E, n=flat.numel(), slots=slots, order=order.to(torch.int32),
                      inv=inv.to(torch.int32), offsets=offsets.to(torch.int32))


# --------------------------------------------------------------------------- pointwise


def rmsnorm(x: Tensor, weight: Tensor, eps: float, out_dtype: torch.dtype) -> Tensor:
    """``x * rsqrt(mean(x^2) + eps) * weight`` with fp32 statistics, rounded to ``out_dtype`` last."""

    x32 = x.float()
    y = x32 * torch.rsqrt(x32.pow(2).mean(dim=-1, keepdim=True) + eps)
    return (y * weight.float()).to(out_dtype)


def grad_sink(x: Tensor) -> Tensor:
    """Identity. The kernel path uses this point to collect the gradients of a depth source that is
    read by many depth reads in one buffer; plain autograd needs no help."""

    return x


class DepthKeyCache:
    """Key scales ``r_i = rsqrt(mean(s_i^2) + eps)`` of depth sources that many reads share.

    The key map of a depth read has no learnable weight, so a source's scale does not depend on the read: every
    sublayer read of a forward pass sees the same embedding and completed-block sources and only its own tail
    changes. The cache holds the leading sources (by object identity) and their scales, computed lazily once and
    reused by every ``depth_read(..., key_cache=cache)``; the list grows with ``extend`` as blocks complete. Pure
    common-subexpression elimination: results are bit-identical to uncached reads (reference
    ``nestor/backbones/attention_residual.py:171-256``). The fused GPU kernel recomputes the scale inside its single
    pass over the sources (it is free there), so the cache serves the PyTorch statement of the op (CPU / evaluation).
    """

    def __init__(self, sources: list[Tensor] | tuple = (), *, eps: float = 1e-6) -> None:
        self.sources = list(sources)
        self.eps = float(eps)
        self._scales: list[Tensor] = []
        self.computed = 0           # how many scale reductions the cache has run (for tests and accounting)

    @property
    def num_sources(self) -> int:
        return len(self.sources)

    def extend(self, sources) -> None:
        self.sources.extend(sources)

    def scales(self) -> list[Tensor]:
        for s in self.sources[len(self._scales):]:
            self._scales.append(torch.rsqrt(s.float().pow(2).mean(dim=-1) + self.eps))
            self.computed += 1
        return self._scales


def depth_read(sources: list[Tensor], query: Tensor, gains: Tensor, eps: float = 1e-6,
               key_cache: DepthKeyCache | None = None) -> Tensor:
    """Softmax-over-depth mixture of unit-RMS sources (fp32).

    ``r_i = rsqrt(mean(s_i^2) + eps)``, ``z_i = r_i (s_i . q) / sqrt(d)``,
    ``w = softmax_i(z) * gain_i``, ``out = sum_i (w_i r_i) s_i``. Sources are ``[..., d]``. ``key_cache`` supplies the
    scales of the leading sources (which must be the very tensors it holds). A two-dimensional ``query [n_max, d]``
    scores source ``i`` with its own row ``q_i``.
    """

    d = sources[0].shape[-1]
    n = len(sources)
    q = query.float()
    cached: list[Tensor] = []
    if key_cache is not None:
        if key_cache.eps != eps:
            raise ValueError("the key cache was built with a different epsilon than this read")
        if key_cache.num_sources > n or any(a is not b for a, b in zip(key_cache.sources, sources)):
            raise ValueError("the leading sources of a cached read must be the cache's own tensors, in order")
        cached = key_cache.scales()[: key_cache.num_sources]
    r, z = [], []
    for i, s in enumerate(sources):
        s32 = s.float()
        ri = cached[i] if i < len(cached) else torch.rsqrt(s32.pow(2).mean(dim=-1) + eps)
        r.append(ri)
        z.append(ri * (s32 @ (q if q.dim() == 1 else q[i])))
    r_all = torch.stack(r, dim=-1)
    w = torch.softmax(torch.stack(z, dim=-1) / math.sqrt(d), dim=-1) * gains[:n].float()
    alpha = w * r_all
    out = sources[0].float() * alpha[..., 0:1]
    for i in range(1, n):
        out = out + sources[i].float() * alpha[..., i : i + 1]
    return out


def depth_attention(values: list[Tensor], query: Tensor, key_gain: Tensor, eps: float = 1e-6) -> Tensor:
    """Attention over a block's sublayer history (``residual_mode='attn_res'``): ``values[0]`` is the block input and
    every later entry one sublayer update, each ``[T, d]``. The logit of entry ``i`` is the pseudo-query ``query [d]``
    against its gain-only RMSNorm, ``z_i = ((q * g) . v_i) * rsqrt(mean(v_i^2) + eps)``; the output is the fp32
    softmax-over-history mixture of the raw values (reference ``nestor/backbones/nestor.py:3900-4074``). Unlike
    :func:`depth_read` the mixture uses the raw values (no unit-RMS rescale), has no per-entry gains and no
    ``1/sqrt(d)`` temperature."""

    w = (query.float().reshape(-1) * key_gain.float())
    z = torch.stack([(v.float() @ w) * torch.rsqrt(v.float().pow(2).mean(dim=-1) + eps) for v in values], dim=-1)
    alpha = torch.softmax(z, dim=-1)
    out = values[0].float() * alpha[..., 0:1]
    for i in range(1, len(values)):
        out = out + values[i].float() * alpha[..., i : i + 1]
    return out


def depth_read_norm(sources: list[Tensor], query: Tensor, gains: Tensor, gamma: Tensor, eps_read: float,
                    eps_norm: float, out_dtype: torch.dtype, key_cache: DepthKeyCache | None = None) -> Tensor:
    """``rmsnorm(depth_read(sources))``: the input of every attention / expert half and of the head."""

    return rmsnorm(depth_read(sources, query, gains, eps_read, key_cache), gamma, eps_norm, out_dtype)


def mid_source(running: Tensor | None, attn: Tensor) -> Tensor:
    """Source of the expert-half read: ``running + mean_j attn[:, j]`` (``[T, d]`` fp32)."""

    m = attn.float().mean(dim=1)
    return m if running is None else running + m


def layer_combine(attn: Tensor, priv: Tensor | None, pub: Tensor, path: Tensor | None, streams: Tensor | None,
                  running: Tensor | None, cd: torch.dtype) -> tuple[Tensor, Tensor]:
    """Add one layer's updates to the column streams and their running mean.

    ``update[t, j] = attn[t, j] + round_cd(path[t, 1] * priv[t, j]) + round_cd(path[t, 0] * pub[t])`` (the path
    weights and ``priv`` are absent for bank / dense layers); ``streams += update``;
    ``running += mean_j update``. Everything is fp32 except the two rounded products.
    """

    if path is not None:
        pubv = (path[:, 0:1].float() * pub.float()).to(cd).float()
        privv = None if priv is None else (path[:, 1:2].float().unsqueeze(-1) * priv.float()).to(cd).float()
    else:
        pubv, privv = pub.float(), None if priv is None else priv.float()
    update = attn.float() + pubv.unsqueeze(1)
    if privv is not None:
        update = update + privv
    streams = update if streams is None else streams + update
    step = update.mean(dim=1)
    return streams, (step if running is None else running + step)


def block_exit(streams: Tensor) -> tuple[Tensor, Tensor]:
    """``(deviations [k, T, d], aggregate [T, d])`` of a block's column streams ``[T, k, d]``."""

    agg = streams.mean(dim=1)
    return (streams - agg.unsqueeze(1)).permute(1, 0, 2), agg


def rope_tables(pos: Tensor, head_dim: int, base: float) -> tuple[Tensor, Tensor]:
    """cos/sin ``[n, head_dim/2]`` in fp32 for integer positions."""

    inv_freq = 1.0 / (base ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=pos.device) / head_dim))
    ang = pos.to(torch.float32).unsqueeze(-1) * inv_freq
    return ang.cos(), ang.sin()


def apply_rope(x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
    """Rotate-half RoPE in fp32 on ``x [n, H, hd]`` with tables ``[n, hd/2]``; returns ``x.dtype``."""

    x32 = x.float()
    half = x.shape[-1] // 2
    x1, x2 = x32[..., :half], x32[..., half:]
    c, s = cos.unsqueeze(1), sin.unsqueeze(1)
    return torch.cat((x1 * c - x2 * s, x2 * c + x1 * s), dim=-1).to(x.dtype)


# ------------------------------------------------------------------------------ router


def router_scores(x: Tensor, w1: Tensor | None, w2: Tensor, cd: torch.dtype) -> Tensor:
    """Score head: a single matrix ``x @ w2^T`` or the MLP ``gelu(x @ w1^T) @ w2^T`` (in ``cd``)."""

    h = x.to(cd)
    if w1 is not None:
        h = F.gelu(h @ w1.to(cd).t())
    return h @ w2.to(cd).t()


class RoutingTape:
    """Record the top-k selections of a forward pass, or replay recorded ones.

    Discrete routing makes two numerically different executions of the same model (kernels
    vs. oracle, recompute vs. first pass) incomparable as soon as one near-tie flips.
    Replaying a tape pins the selections so only the continuous math differs.
    """

    def __init__(self) -> None:
        self.selections: list[Tensor] = []
        self.cursor = 0
        self.mode: str | None = None


_TAPE: RoutingTape | None = None


def set_routing_tape(tape: RoutingTape | None, mode: str | None = None) -> None:
    """``mode``: ``"record"``, ``"replay"`` or ``None`` (tape off)."""

    global _TAPE
    _TAPE = tape if mode else None
    if tape is not None:
        tape.mode = mode
        tape.cursor = 0
        if mode == "record":
            tape.selections = []


def route_topk(scores: Tensor, bias: Tensor, k: int, gate_mode: str) -> tuple[Tensor, Tensor]:
    """Top-k on ``scores + bias``; gates from the raw scores.

    ``renorm``: softmax over the ``k`` selected raw scores. ``switch``: the selected
    entries of the full softmax. Gates are fp32. Returns ``(idx [.., k], gates [.., k])``.
    """

    if _TAPE is not None and _TAPE.mode == "replay":
        idx = _TAPE.selections[_TAPE.cursor]
        _TAPE.cursor += 1
    else:
        idx = torch.topk(scores.float() + bias.float(), k=k, dim=-1).indices
        if _TAPE is not None and _TAPE.mode == "record":
            _TAPE.selections.append(idx)
    if gate_mode == "switch":
        gates = torch.softmax(scores.float(), dim=-1).gather(-1, idx)
    else:
        gates = torch.softmax(scores.float().gather(-1, idx), dim=-1)
    return idx, gates


def route_selected(scores: Tensor, bias: Tensor, cols: Tensor, col_gates: Tensor, k: int, gate_mode: str,
                   cd: torch.dtype) -> tuple[Tensor, Tensor, Tensor]:
    """Private-expert routing inside the selected columns.

    ``scores [T, G, Q]`` holds every column's private-router scores, ``bias [G, Q]`` their selection
    biases, ``cols [T, kc]`` the columns a token was routed to and ``col_gates [T, kc]`` their gates.
    Each (token, selected column) pair picks ``k`` of that column's ``Q`` experts (``route_topk``).
    Returns ``(expert ids [T, kc*k]`` (``column * Q + choice``), ``weights [T, kc*k]`` in ``cd``
    (``gate.to(cd) * col_gate.to(cd)``), ``choices [T, kc, k])``.
    """

    T, G, Q = scores.shape
    col = cols.long()
    sel_scores = scores.gather(1, col.unsqueeze(-1).expand(-1, -1, Q))          # [T, kc, Q]
    idx, gate = route_topk(sel_scores, bias[col], k, gate_mode)                 # [T, kc, k]
    ids = (col.unsqueeze(-1) * Q + idx).reshape(T, -1)
    w = (gate.to(cd) * col_gates.to(cd).unsqueeze(-1)).reshape(T, -1)
    return ids, w, idx


# ---------------------------------------------------------------------------- attention


def causal_attention(q: Tensor, k: Tensor, v: Tensor, scale: float, causal: bool = True) -> Tensor:
    """Softmax attention on ``[n, H, hd]`` (one segment), causal unless told otherwise; fp32 softmax, output in
    ``q.dtype``."""

    n = q.shape[0]
    if n == 0:
        return q.new_zeros(q.shape)
    qh, kh, vh = (t.transpose(0, 1) for t in (q, k, v))
    s = (qh.float() @ kh.float().transpose(1, 2)) * scale
    if causal:
        mask = torch.ones(n, n, dtype=torch.bool, device=q.device).tril()
        s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, dim=-1)
    return (p.to(q.dtype).float() @ vh.float()).to(q.dtype).transpose(0, 1)


def segment_attention(q: Tensor, k: Tensor, v: Tensor, seg_start: Tensor, scale: float, causal: bool = True) -> Tensor:
    """Attention independently inside each packed segment (causal by default). ``q/k/v [rows, H, hd]``."""

    out = torch.empty_like(q)
    bounds = seg_start.tolist()
    for a, b in zip(bounds[:-1], bounds[1:]):
        if b > a:
            if q.is_cuda:
                o = F.scaled_dot_product_attention(
                    q[a:b].transpose(0, 1).unsqueeze(0), k[a:b].transpose(0, 1).unsqueeze(0),
                    v[a:b].transpose(0, 1).unsqueeze(0), is_causal=causal, scale=scale)
                out[a:b] = o.squeeze(0).transpose(0, 1)
            else:
                out[a:b] = causal_attention(q[a:b], k[a:b], v[a:b], scale, causal)
    return out


def column_attention(
    n: Tensor, plan: ColumnPlan, gates: Tensor, wqkv: Tensor, wo: Tensor,
    heads: int, head_dim: int, rope_base: float, cd: torch.dtype, causal: bool = True,
) -> Tensor:
    """Column-routed causal attention: ``[T, d] -> [T, k, d]`` gated slot updates (fp32). ``causal=False`` lets every
    member of a column see all members of its sequence (bidirectional encoders).

    ``wqkv [G, 3*inner, d]`` stacks each column's ``q_proj, k_proj, v_proj`` rows; ``wo [G, d, inner]``.
    For every column ``c``: project its member rows, RoPE at the rows' original positions,
    causal attention among the members of each sequence with logits scaled by
    ``1 / head_dim``, project with ``wo[c]``, multiply by the token's gate for ``c`` and place
    the result in the slot that owns ``c``. ``gates`` is ``[T, k]`` in slot order.
    """

    T, d = n.shape
    inner = heads * head_dim
    x = n.to(cd)[plan.tok_of_row.long()]                       # pack: [rows, d]
    cos, sin = rope_tables(plan.pos_of_row, head_dim, rope_base)
    qkv = x.new_empty(plan.rows, 3 * inner)
    cs = plan.col_start.tolist()
    for c in range(plan.G):
        a, b = cs[c], cs[c + 1]
        qkv[a:b] = x[a:b] @ wqkv[c].to(cd).t()
    q = apply_rope(qkv[:, :inner].reshape(-1, heads, head_dim), cos, sin)
    kk = apply_rope(qkv[:, inner : 2 * inner].reshape(-1, heads, head_dim), cos, sin)
    v = qkv[:, 2 * inner :].reshape(-1, heads, head_dim)
    o = segment_attention(q, kk, v, plan.seg_start, 1.0 / head_dim, causal).reshape(plan.rows, inner)
    y = x.new_empty(plan.rows, d)
    for c in range(plan.G):
        a, b = cs[c], cs[c + 1]
        y[a:b] = o[a:b] @ wo[c].to(cd).t()
    upd = y[plan.row_of_slot.long().reshape(-1)].view(T, plan.k, d).float()
    return upd * gates.float().unsqueeze(-1)


def dense_attention(
    n: Tensor, B: int, S: int, wqkv: Tensor, wo: Tensor,
    heads: int, head_dim: int, rope_base: float, cd: torch.dtype, pos: Tensor | None = None, causal: bool = True,
) -> Tensor:
    """Single-column causal MHA over whole sequences: ``[T, d] -> [T, d]`` (baseline arms); ``causal=False`` is full
    bidirectional attention.

    ``wqkv [1, 3*inner, d]`` (``q_proj, k_proj, v_proj`` rows), ``wo [1, d, inner]``.
    """

    wqkv, wo = wqkv[0], wo[0]
    T, d = n.shape
    inner = heads * head_dim
    x = n.to(cd)
    p = torch.arange(S, device=n.device).repeat(B) if pos is None else pos.reshape(-1).clamp_min(0)
    cos, sin = rope_tables(p, head_dim, rope_base)
    qkv = x @ wqkv.to(cd).t()
    q = apply_rope(qkv[:, :inner].reshape(T, heads, head_dim), cos, sin)
    k = apply_rope(qkv[:, inner : 2 * inner].reshape(T, heads, head_dim), cos, sin)
    v = qkv[:, 2 * inner :].reshape(T, heads, head_dim)
    seg = torch.arange(0, T + 1, S, device=n.device, dtype=torch.int32)
    o = segment_attention(q, k, v, seg, 1.0 / head_dim, causal).reshape(T, inner)
    return (o @ wo.to(cd).t()).float()


# ------------------------------------------------------------------------------ experts


def swiglu(gate: Tensor, up: Tensor) -> Tensor:
    """``silu(gate) * up`` with the product formed after rounding ``silu`` to the input dtype."""

    return F.silu(gate) * up


POINTWISE_ACTIVATIONS = {"relu": F.relu, "gelu": F.gelu, "silu": F.silu, "tanh": torch.tanh}


def expert_bank(
    x: Tensor, plan: ExpertPlan, weights: Tensor, w_up: Tensor, w_gate: Tensor | None, w_down: Tensor,
    cd: torch.dtype, group: int, activation: str = "swiglu",
) -> Tensor:
    """Routed SwiGLU bank: ``[T, d] -> [T, slots/group, d]`` (fp32).

    Banks are stacked ``w_up, w_gate [E, d, h]``, ``w_down [E, h, d]``. Slot ``s`` of token
    ``t`` runs expert ``ids[t, s]``; the outputs of each run of ``group`` consecutive slots
    are summed with their ``weights [T, slots]`` (each product rounded to ``cd`` before
    the fp32 sum). A pointwise ``activation`` (``relu / gelu / silu / tanh``) takes no gate bank: the hidden row is
    ``act(x @ w_up)``.
    """

    T, d = x.shape
    xs = x.to(cd)[(plan.order.long() // plan.slots)]            # dispatch gather [n, d]
    y = xs.new_empty(plan.n, d)
    off = plan.offsets.tolist()
    for e in range(plan.E):
        a, b = off[e], off[e + 1]
        if b > a:
            up = xs[a:b] @ w_up[e].to(cd)
            h = swiglu(xs[a:b] @ w_gate[e].to(cd), up) if activation == "swiglu" else POINTWISE_ACTIVATIONS[activation](up)
            y[a:b] = h @ w_down[e].to(cd)
    per_slot = y[plan.inv.long()].view(T, plan.slots, d)
    weighted = (per_slot.float() * weights.float().unsqueeze(-1)).to(cd)
    return weighted.view(T, plan.slots // group, group, d).float().sum(dim=2)


def dense_swiglu(x: Tensor, w_up: Tensor, w_gate: Tensor | None, w_down: Tensor, cd: torch.dtype,
                 activation: str = "swiglu") -> Tensor:
    """One SwiGLU MLP with ``nn.Linear``-layout weights (``[h, d]``, ``[h, d]``, ``[d, h]``); with a pointwise
    ``activation`` the MLP is ``act(x @ w_up^T) @ w_down^T`` and takes no gate."""

    h = x.to(cd)
    up = h @ w_up.to(cd).t()
    hidden = swiglu(h @ w_gate.to(cd).t(), up) if activation == "swiglu" else POINTWISE_ACTIVATIONS[activation](up)
    return (hidden @ w_down.to(cd).t()).float()


# --------------------------------------------------------------------------------- head


def lm_head_ce(hidden: Tensor, weight: Tensor, targets: Tensor, multiplier: float, cd: torch.dtype,
               chunk_rows: int = 4096, ignore_index: int = -100) -> tuple[Tensor, Tensor]:
    """Summed cross-entropy of ``(hidden @ weight^T) * multiplier`` against ``targets``.

    Never holds more than ``chunk_rows x V`` logits; log-sum-exp in fp32. Returns
    ``(loss_sum, num_valid)`` as fp32 / int64 scalars (tensors, no host sync).
    """

    from torch.utils.checkpoint import checkpoint

    def chunk(h: Tensor, t: Tensor, w32: Tensor) -> Tensor:
        logits = (h.to(cd) @ w32.to(cd).t()) * multiplier
        return F.cross_entropy(logits.float(), t, ignore_index=ignore_index, reduction="sum")

    total = hidden.new_zeros((), dtype=torch.float32)
    recompute = torch.is_grad_enabled() and (hidden.requires_grad or weight.requires_grad)
    for a in range(0, hidden.shape[0], chunk_rows):
        h, t = hidden[a : a + chunk_rows], targets[a : a + chunk_rows]
        total = total + (checkpoint(chunk, h, t, weight, use_reentrant=False) if recompute else chunk(h, t, weight))
    return total, (targets != ignore_index).sum()


# ------------------------------------------------------------------------ Newton–Schulz

NS_COEFFS = (3.4445, -4.7750, 2.0315)


def newton_schulz(g: Tensor, steps: int = 5, out_dtype: torch.dtype | None = None) -> Tensor:
    """Quintic Newton–Schulz orthogonalisation of ``[..., m, n]`` matrices in bf16.

    Normalise by the Frobenius norm (+1e-7), work on the wide orientation, iterate
    ``A = X X^T; B = bA + cA^2; X = aX + BX``.
    """

    a, b, c = NS_COEFFS
    squeeze = g.ndim == 2
    x = (g.unsqueeze(0) if squeeze else g).bfloat16()
    transposed = x.size(-2) > x.size(-1)
    if transposed:
        x = x.mT
    x = x / (x.norm(dim=(-2, -1), keepdim=True) + 1e-7)
    for _ in range(steps):
        aa = x @ x.mT
        bb = b * aa + c * (aa @ aa)
        x = a * x + bb @ x
    if transposed:
        x = x.mT
    x = x.to(g.dtype if out_dtype is None else out_dtype)
    return x.squeeze(0) if squeeze else x
