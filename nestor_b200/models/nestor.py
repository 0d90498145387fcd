"""The Nestor decoder: blocks of column-routed attention + expert MLPs joined by depth reads.

Forward semantics follow the reference's registered-experiment path
(``nestor/backbones/nestor.py``: block ``:9295-9642``, column layer ``:7327-7533`` and
``:7804-7909``, Kimi layer ``:6952-7034``, backbone ``:10244-10440``):

* A block runs its group router once; slot ``j`` of a token owns column ``idx[j]`` for
  the whole block. Each token carries ``k`` residual streams plus their running mean.
* A column layer reads ``h = DepthRead([x0, agg_1.., running])``, normalises, runs
  column attention into the ``k`` slots, reads again with ``running + mean(attn)``,
  normalises, runs the hybrid expert pool (private experts per slot, public experts
  broadcast), and adds both updates to the streams with no residual multiplier.
* A block exports its ``k`` deviations ``s_j - agg`` and the aggregate ``agg``; sublayer
  reads see only the aggregates, the final head read sees every export.
* Baseline (Kimi) blocks are the single-column special case with a plain running sum.

Beside that path the block also runs the reference's other topologies: the merged recurrence for multi-column
blocks that keep no streams (``Block._merged_layers``: ``attn_res_kimi``, blocks left out of
``block_column_blocks``, the leading layers under ``block_column_trailing_layers``), column-resolved sublayer reads
(``Block._forward_wide_reads``), the plain residual stream (``Block._forward_projection``) and the within-block
history attention (``Block._forward_history_attention``); causal or bidirectional attention; pools or banks (shared
and column-specific experts, gated or pointwise).

All tensors are flattened to ``[T, ...]`` with ``T = B * S``; residual streams are fp32
and matrix products run in the compute dtype ``cd``.
"""

from __future__ import annotations

import os

import math
from typing import Any

import torch
from torch import Tensor, nn

from nestor_b200 import ops
from nestor_b200.configs.model import BlockSpec, NestorConfig, ReferenceMupConfig
from nestor_b200.models.modules import (
    BlockAttentionResidual, ColumnProjections, DenseExpert, DepthRead, ExpertBank, Matrix, Norm, RouterParams,
)
from nestor_b200.models.registry import Backbone
from nestor_b200.models.tags import ADAMW_DECAY


def W(owner: nn.Module, p: Tensor) -> Tensor:
    """Weight operand of ``p``: the arena's compute-dtype view when the model is arena-backed."""

    arena = owner.__dict__.get("_nestor_arena")
    return p if arena is None or not p.requires_grad else arena.compute_view(p)


def Wstack(owner: nn.Module, params: list[Tensor]) -> Tensor:
    """``[n, ...]`` operand over same-shape parameters (a strided arena view when possible)."""

    arena = owner.__dict__.get("_nestor_arena")
    if arena is None or not params[0].requires_grad:
        return torch.stack(list(params), dim=0)
    return arena.stack_view(params)


class InitScales:
    """Initialisation constants of one model (reference muP: ``reference_mup.py:126-127``)."""

    def __init__(self, mup: ReferenceMupConfig | None, dim: int, total_layers: int) -> None:
        if mup is not None:
            self.matrix = mup.initializer_range / math.sqrt(mup.width_multiplier)
            self.output = self.matrix / math.sqrt(2 * mup.num_layers)
            self.router = self.matrix
            self.table = mup.initializer_range
            self.norm_eps = mup.norm_eps
        else:
            self.matrix = 1.0 / math.sqrt(dim)
            self.output = self.matrix / math.sqrt(2 * total_layers)
            self.router = self.matrix
            self.table = 1.0
            self.norm_eps = 1e-6


class _SplitColumns(torch.autograd.Function):
    """Contiguous column blocks of a ``[T, C]`` matrix. Plain slices would each send a zero-filled ``[T, C]`` gradient
    back (a fill, a copy and an add per slice); here the blocks' gradients are concatenated once."""

    @staticmethod
    def forward(ctx, x: Tensor, sizes: tuple[int, ...]):
        ctx.sizes, ctx.dtype = sizes, x.dtype
        return tuple(part.contiguous() for part in torch.split(x, list(sizes), dim=1))

    @staticmethod
    def backward(ctx, *grads):
        T = next(g for g in grads if g is not None).shape[0]
        dev = next(g for g in grads if g is not None).device
        parts = [g.to(ctx.dtype) if g is not None else torch.zeros(T, n, dtype=ctx.dtype, device=dev)
                 for g, n in zip(grads, ctx.sizes)]
        return torch.cat(parts, dim=1), None


class ExpertPool(nn.Module):
    """Hybrid pool: ``P`` public experts + ``Q`` private experts per column + 2-logit path gate.

    ``P == 0`` is the private-only pool (reference ``nestor/backbones/expert_pools.py:23-29,1102-1104``): every column
    draws from its own private experts only; no public router, public bank or path gate exists, and the private
    path's weight is the constant 1.
    """

    def __init__(self, s: BlockSpec, init: InitScales) -> None:
        super().__init__()
        self.spec = s
        mk = lambda c, k, mode: RouterParams(  # noqa: E731
            s.dim, c, k, std=init.router, gate_mode=mode, loss_free=s.loss_free, bias_rate=s.bias_rate)
        self.has_public = s.P > 0
        self.public_router = mk(s.P, s.k_p, "renorm") if self.has_public else None
        self.private_routers = nn.ModuleList([mk(s.Q, s.k_q, s.private_gate) for _ in range(s.G)])
        self.path_gate = Matrix(s.dim, 2, ADAMW_DECAY, init.matrix) if self.has_public else None
        self.stacked_public = ExpertBank(s.P, s.dim, s.h_pub, init.matrix, init.output) if self.has_public else None
        self.stacked_private = ExpertBank(s.G * s.Q, s.dim, s.h_priv, init.matrix, init.output)

    def private_router_weight(self) -> Tensor:
        """``[G*Q, d]``: the ``G`` single-matrix private routers stacked (one batched GEMM)."""

        w = Wstack(self, [r.score_mlp.layers[0].weight for r in self.private_routers])
        return w.reshape(-1, w.shape[-1])

    def private_bias(self) -> Tensor:
        return torch.stack([r.choice_bias for r in self.private_routers], dim=0)

    def forward(self, n: Tensor, idx: Tensor, gates: Tensor, cd: torch.dtype) -> tuple[Tensor, Tensor, Tensor, dict]:
        """``n [T, d]`` -> ``(public [T, d], private [T, k, d], path [T, 2], aux)``; the path weights are
        applied when the layer's updates are combined into the streams."""

        s = self.spec
        T = n.shape[0]
        # one GEMM for the public router, the G private routers and the path gate (adjacent parameters)
        if not self.has_public:
            return self._forward_private_only(n, idx, gates, cd)
        heads = [self.public_router.score_mlp.layers[0].weight,
                 *[r.score_mlp.layers[0].weight for r in self.private_routers], self.path_gate.weight]
        arena = self.__dict__.get("_nestor_arena")
        wcat = arena.concat_view(heads) if arena is not None and heads[0].requires_grad else torch.cat(heads, dim=0)
        scores = ops.router_scores(n, None, wcat, cd)
        pub_scores, priv_scores, path_logits = _SplitColumns.apply(scores, (s.P, s.G * s.Q, 2))
        priv_scores = priv_scores.view(T, s.G, s.Q)
        pub_idx, pub_gate = ops.route_topk(pub_scores, self.public_router.choice_bias, s.k_p, "renorm")
        # every (token, selected column) pair picks k_q of that column's Q private experts
        priv_ids, priv_w, priv_idx = ops.route_selected(priv_scores, self.private_bias(), idx, gates, s.k_q,
                                                        s.private_gate, cd)
        path = torch.softmax(path_logits.float(), dim=-1)

        pub_plan = ops.build_expert_plan(pub_idx, s.P)
        public = ops.expert_bank(n, pub_plan, pub_gate.to(cd), W(self, self.stacked_public.w_up),
                                 W(self, self.stacked_public.w_gate), W(self, self.stacked_public.w_down), cd, group=s.k_p)
        priv_plan = ops.build_expert_plan(priv_ids, s.G * s.Q)
        private = ops.expert_bank(n, priv_plan, priv_w, W(self, self.stacked_private.w_up),
                                  W(self, self.stacked_private.w_gate), W(self, self.stacked_private.w_down), cd, group=s.k_q)
        aux = {"public_idx": pub_idx, "private_idx": priv_idx, "columns": idx,
               "public_offsets": pub_plan.offsets, "private_offsets": priv_plan.offsets}
        if not self.training and not torch.is_grad_enabled():
            # evaluation only: soft routing mass per choice (the reference's ``prob/*`` metrics). A private router's
            # mass counts the tokens routed into its column.
            aux["public_prob"] = torch.softmax(pub_scores.float(), dim=-1).sum(0)
            member = torch.zeros(T, s.G, device=n.device).scatter_(1, idx.long(), 1.0)
            aux["private_prob"] = (torch.softmax(priv_scores.float(), dim=-1) * member.unsqueeze(-1)).sum(0)
        return public.view(T, s.dim), private, path, aux      # [T, 1, d] -> [T, d] as a view (a select would zero-fill in backward)

    def _forward_private_only(self, n: Tensor, idx: Tensor, gates: Tensor, cd: torch.dtype):
        """No public path and no path gate: ``(zeros [T, d], private [T, k, d], None, aux)``."""

        s = self.spec
        T = n.shape[0]
        scores = ops.router_scores(n, None, self.private_router_weight(), cd).reshape(T, s.G, s.Q)
        priv_ids, priv_w, priv_idx = ops.route_selected(scores, self.private_bias(), idx, gates, s.k_q, s.private_gate, cd)
        plan = ops.build_expert_plan(priv_ids, s.G * s.Q)
        private = ops.expert_bank(n, plan, priv_w, W(self, self.stacked_private.w_up), W(self, self.stacked_private.w_gate),
                                  W(self, self.stacked_private.w_down), cd, group=s.k_q)
        aux = {"private_idx": priv_idx, "columns": idx, "private_offsets": plan.offsets}
        if not self.training and not torch.is_grad_enabled():
            member = torch.zeros(T, s.G, device=n.device).scatter_(1, idx.long(), 1.0)
            aux["private_prob"] = (torch.softmax(scores.float(), dim=-1) * member.unsqueeze(-1)).sum(0)
        return torch.zeros(T, s.dim, dtype=cd, device=n.device), private, None, aux


class Layer(nn.Module):
    """One transformer layer (attention half + expert half) of a block."""

    def __init__(self, s: BlockSpec, init: InitScales, max_sources: int, dense_no_router: bool,
                 depth_reads: bool = True, drop_path: float = 0.0, bank_experts: int | None = None,
                 history_attention: bool = False) -> None:
        super().__init__()
        self.spec = s
        if history_attention:
            # residual_mode='attn_res': a zero-initialised pseudo-query and a gain-only key norm per sublayer
            # (reference nestor/backbones/nestor.py:4282-4295)
            from nestor_b200.models.scaling import ScaledLinear
            self.attn_query = ScaledLinear(s.dim, 1, role="score", bias=False, zero_init=True)
            self.attn_key_norm = Norm(s.dim, init.norm_eps)
            self.mlp_query = ScaledLinear(s.dim, 1, role="score", bias=False, zero_init=True)
            self.mlp_key_norm = Norm(s.dim, init.norm_eps)
        self.bank_experts = E = s.bank_experts if bank_experts is None else bank_experts   # this layer's router choices
        # Choices past the shared ones name one expert PER COLUMN: the stacked bank is [shared | column 0 | column 1 ...]
        # (reference nestor/backbones/nestor.py:4419-4436, 4456-4470). With one column they are plain further experts.
        self.bank_specific = E - s.bank_shared if (s.G > 1 and not s.pool and s.bank_shared is not None) else 0
        bank_total = E + (s.G - 1) * self.bank_specific
        gated = s.activation == "swiglu"      # pointwise activations: experts without a gate matrix
        self.attn_norm = Norm(s.dim, init.norm_eps)
        self.mlp_norm = Norm(s.dim, init.norm_eps)
        self.drop_path = float(os.environ.get("NESTOR_DROP_PATH_RATE") or drop_path)
        if depth_reads:
            self.kimi_attn_read = DepthRead(s.dim, max_sources)
            self.kimi_mlp_read = DepthRead(s.dim, max_sources)
        self.attention_groups = nn.ModuleList(
            [ColumnProjections(s.dim, s.inner, init.matrix, init.output) for _ in range(s.G)])
        self.expert_pool: ExpertPool | None = None
        self.expert_router: RouterParams | None = None
        self.stacked_moe_bank: ExpertBank | None = None
        self.shared_experts: nn.ModuleList | None = None
        if s.pool:
            self.expert_pool = ExpertPool(s, init)
        else:
            self.expert_router = RouterParams(
                s.dim, E, s.bank_top_k, std=init.router,
                loss_free=s.loss_free, bias_rate=s.bias_rate)
            if E == 1:
                # A one-choice gate is the constant 1.0: the router can never receive a
                # gradient, so it is frozen (and, with dense_no_router, skipped entirely).
                self.expert_router.requires_grad_(False)
                self.shared_experts = nn.ModuleList([DenseExpert(s.dim, s.bank_width, init.matrix, init.output, gated)])
            else:
                self.stacked_moe_bank = ExpertBank(bank_total, s.dim, s.bank_width, init.matrix, init.output, gated)
        # DeepSeekMoE-style always-on experts beside a routed bank: every token, unit gate, outside the router
        # (reference nestor/backbones/nestor.py:4441-4451, 5290-5291)
        self.dense_shared_experts = nn.ModuleList(
            [DenseExpert(s.dim, s.bank_width, init.matrix, init.output, gated) for _ in range(0 if s.pool else s.dense_shared)])
        self.dense_no_router = dense_no_router

    # -- weight views ---------------------------------------------------------------
    def qkv_weight(self) -> Tensor:
        """``[G, 3*inner, d]``: every column's ``q_proj, k_proj, v_proj`` rows, one operand."""

        groups = [[g.q_proj.weight, g.k_proj.weight, g.v_proj.weight] for g in self.attention_groups]
        arena = self.__dict__.get("_nestor_arena")
        if arena is not None and groups[0][0].requires_grad:
            return arena.fused_view(groups)
        return torch.stack([torch.cat(g, dim=0) for g in groups], dim=0)

    def out_weight(self) -> Tensor:
        return Wstack(self, [g.out_proj.weight for g in self.attention_groups])

    def drop(self, update: Tensor, B: int) -> Tensor:
        """Stochastic depth on a sublayer update (per sequence, survivors rescaled by ``1 / keep``): training only
        (reference ``nestor/backbones/nestor.py:4891-4910``)."""

        p = self.drop_path
        if p <= 0.0 or not self.training:
            return update
        keep = 1.0 - p
        mask = (torch.rand(B, device=update.device) < keep).to(update.dtype) / keep
        rows = update.shape[0] // B
        return update * mask.repeat_interleave(rows).view(-1, *([1] * (update.dim() - 1)))

    # -- halves -----------------------------------------------------------------------
    def attention(self, n: Tensor, ctx: "BlockContext", cd: torch.dtype) -> Tensor:
        s = self.spec
        if s.G == 1:
            extra = {} if s.causal else {"causal": False}
            out = ops.dense_attention(n, ctx.B, ctx.S, self.qkv_weight(), self.out_weight(),
                                      s.heads, s.head_dim, s.rope_base, cd, pos=ctx.pos, **extra)
            return out.unsqueeze(1)
        extra = {} if s.causal else {"causal": False}
        return ops.column_attention(n, ctx.plan, ctx.gates, self.qkv_weight(), self.out_weight(),
                                    s.heads, s.head_dim, s.rope_base, cd, **extra)

    def attention_step(self, n: Tensor, ctx: "BlockContext", cd: torch.dtype, cache: "LayerKVCache") -> Tensor:
        """Attention half for ONE new token per sequence (``n [B, d]``) against this layer's key/value cache.

        Slot ``j`` of sequence ``b`` projects with the weights of column ``idx[b, j]``, appends its rotated key and its
        value to that column's cache and attends over everything the column has seen of the sequence so far, which
        is exactly the causal row the full forward computes for that token (the members of a column are visited in
        position order). Returns the gated slot updates ``[B, k, d]`` in fp32.
        """

        s = self.spec
        B = n.shape[0]
        heads, hd, inner = s.heads, s.head_dim, s.heads * s.head_dim
        wqkv, wo = self.qkv_weight().to(cd), self.out_weight().to(cd)            # [G, 3*inner, d], [G, d, inner]
        cos, sin = ops.rope_tables(ctx.pos.reshape(-1).clamp_min(0), hd, s.rope_base)
        x = n.to(cd)
        rows = torch.arange(B, device=n.device)
        out = []
        for j in range(ctx.idx.shape[1]):
            c = ctx.idx[:, j].long()
            qkv = torch.einsum("bd,bnd->bn", x, wqkv[c])
            q = ops.apply_rope(qkv[:, :inner].reshape(B, heads, hd), cos, sin)
            k = ops.apply_rope(qkv[:, inner : 2 * inner].reshape(B, heads, hd), cos, sin)
            v = qkv[:, 2 * inner :].reshape(B, heads, hd)
            at = cache.count[rows, c]
            if int(at.max()) >= cache.keys.shape[2]:
                raise ValueError(f"key/value cache of {cache.keys.shape[2]} positions per column is full")
            cache.keys[rows, c, at] = k.to(cache.keys.dtype)
            cache.values[rows, c, at] = v.to(cache.values.dtype)
            cache.count[rows, c] = at + 1
            K, V = cache.keys[rows, c], cache.values[rows, c]                 # [B, L, H, hd]
            visible = torch.arange(K.shape[1], device=n.device).unsqueeze(0) <= at.unsqueeze(1)
            sc = torch.einsum("bhd,blhd->bhl", q.float(), K.float()) / hd
            p = torch.softmax(sc.masked_fill(~visible.unsqueeze(1), float("-inf")), dim=-1)
            o = torch.einsum("bhl,blhd->bhd", p.to(cd).float(), V.float()).to(cd).reshape(B, inner)
            y = torch.einsum("bi,bdi->bd", o, wo[c]).float()
            out.append(y * ctx.gates[:, j].float().unsqueeze(-1))
        return torch.stack(out, dim=1)

    def experts(self, n: Tensor, ctx: "BlockContext", cd: torch.dtype) -> tuple[Tensor | None, Tensor, Tensor | None, dict]:
        """Expert half: ``(private [T, k, d] | None, shared [T, d], path [T, 2] | None, routing aux)``."""

        s = self.spec
        if self.expert_pool is not None:
            public, private, path, aux = self.expert_pool(n, ctx.idx, ctx.gates, cd)
            return private, public, path, aux
        if self.shared_experts is not None:
            return None, self._add_dense_shared(self._dense_expert(self.shared_experts[0], n, cd), n, cd), None, {}
        scores = ops.router_scores(n, None, W(self, self.expert_router.score_mlp.layers[0].weight), cd)
        idx, gate = ops.route_topk(scores, self.expert_router.choice_bias, s.bank_top_k, "renorm")
        bank = self.stacked_moe_bank
        ids, row_w = idx, gate
        if self.bank_specific:
            # a shared choice is one row; a column-specific choice is one row per selected column, in that column's
            # slice of the bank and weighted by the column gate as well (rows of a shared choice past the first
            # carry weight zero, which keeps every shape static); reference nestor/backbones/nestor.py:4816-4835
            T, k = ctx.idx.shape
            col = ctx.idx.to(idx.dtype)
            specific = (idx >= self.bank_experts - self.bank_specific).unsqueeze(-1)               # [T, top_k, 1]
            ids = torch.where(specific, idx.unsqueeze(-1) + col.unsqueeze(1) * self.bank_specific,
                              idx.unsqueeze(-1).expand(-1, -1, k)).reshape(T, -1)
            first = torch.zeros(k, dtype=gate.dtype, device=gate.device)
            first[0] = 1.0
            row_w = torch.where(specific, gate.unsqueeze(-1) * ctx.gates.to(gate.dtype).unsqueeze(1),
                                gate.unsqueeze(-1) * first).reshape(T, -1)
        plan = ops.build_expert_plan(ids, bank.num_experts)
        ones = torch.ones_like(row_w, dtype=cd)
        if bank.gated:
            rows = ops.expert_bank(n, plan, ones, W(self, bank.w_up), W(self, bank.w_gate), W(self, bank.w_down), cd, group=1)
        else:
            rows = ops.expert_bank(n, plan, ones, W(self, bank.w_up), None, W(self, bank.w_down), cd, group=1,
                                   activation=s.activation)
        out = (rows * row_w.to(cd).float().unsqueeze(-1)).sum(dim=1).to(cd).float()
        aux = {"expert_idx": idx, "expert_router": {"scores": scores, "topk_indices": idx}}
        if not self.training and not torch.is_grad_enabled():
            aux["expert_prob"] = torch.softmax(scores.float(), dim=-1).sum(0)
        return None, self._add_dense_shared(out, n, cd), None, aux

    def _dense_expert(self, e: DenseExpert, n: Tensor, cd: torch.dtype) -> Tensor:
        if e.gated:
            return ops.dense_swiglu(n, W(self, e.layers[0].weight), W(self, e.gate.weight), W(self, e.layers[1].weight), cd)
        return ops.dense_swiglu(n, W(self, e.layers[0].weight), None, W(self, e.layers[1].weight), cd,
                                activation=self.spec.activation)

    def _add_dense_shared(self, out: Tensor, n: Tensor, cd: torch.dtype) -> Tensor:
        for e in self.dense_shared_experts:
            out = out + self._dense_expert(e, n, cd)
        return out


class LayerKVCache:
    """Keys and values one layer has seen, per sequence and column: ``keys / values [B, G, L, H, hd]`` and the number
    of entries ``count [B, G]`` (a token only enters the columns it was routed to, so the counts differ)."""

    def __init__(self, B: int, G: int, max_len: int, heads: int, head_dim: int, device, dtype) -> None:
        self.keys = torch.zeros(B, G, max_len, heads, head_dim, device=device, dtype=dtype)
        self.values = torch.zeros_like(self.keys)
        self.count = torch.zeros(B, G, dtype=torch.long, device=device)


class NestorKVCache:
    """Decode state of the whole backbone: one ``LayerKVCache`` per (block, layer)."""

    def __init__(self, backbone: "Nestor", B: int, max_len: int, device, dtype=torch.float32) -> None:
        self.blocks = [[LayerKVCache(B, blk.spec.G, max_len, blk.spec.heads, blk.spec.head_dim, device, dtype)
                        for _ in blk.layers] for blk in backbone.blocks]
        self.length = 0


class BlockContext:
    """Per-block routing state shared by the block's layers."""

    def __init__(self, B: int, S: int, idx: Tensor, gates: Tensor, plan: Any, pos: Tensor | None) -> None:
        self.B, self.S, self.idx, self.gates, self.plan, self.pos = B, S, idx, gates, plan, pos

    def rows(self, a: int, b: int) -> "BlockContext":
        """The routing state of token rows ``a:b`` (what a per-token op such as the expert half needs)."""

        return BlockContext(self.B, self.S, self.idx[a:b], self.gates[a:b], None, None)


class RecomputeLadder:
    """Which parts of a block are recomputed in the backward pass instead of kept (all exact: the regions are pure
    functions of their tensor arguments, the random state is replayed, the kernels are deterministic).

    Flags, read at every forward (reference ``nestor/backbones/nestor.py:1077-1401``, launcher recipes
    ``scripts/slurm_extend.sh:66-85``):

    * ``NESTOR_ACTIVATION_CHECKPOINT=1``           every layer is a region (keeps ``streams [T, k, d]`` per layer);
    * ``..._CHECKPOINT_SPLIT=1``                   the attention half and the expert half are separate regions;
    * ``..._CHECKPOINT_LEAN=1``                    same split; named for what it keeps: a half's inputs here are the
      ``[T, d]`` sources and running mean only, so split halves are lean by construction;
    * ``..._CHECKPOINT_BLOCK=1``                   the whole block is one outer region (least memory, most recompute);
    * ``NESTOR_EXPERT_HALF_CHUNKS=n``              the expert half runs over ``n`` row chunks, one region each;
    * ``NESTOR_DENSE_TAIL_QUERY_CHUNKS``           accepted for launcher compatibility, no effect: the attention
      kernels never materialise scores, which is what that rung saved.
    """

    def __init__(self, on: bool, split: bool, block: bool, chunks: int) -> None:
        self.on, self.split, self.block, self.chunks = on, split, block, chunks

    @classmethod
    def current(cls, active: bool) -> "RecomputeLadder":
        env = os.environ.get
        on = active and env("NESTOR_ACTIVATION_CHECKPOINT") == "1" and torch.is_grad_enabled()
        split = env("NESTOR_ACTIVATION_CHECKPOINT_SPLIT") == "1" or env("NESTOR_ACTIVATION_CHECKPOINT_LEAN") == "1"
        return cls(on, split, env("NESTOR_ACTIVATION_CHECKPOINT_BLOCK") == "1", int(env("NESTOR_EXPERT_HALF_CHUNKS") or 0))

    @property
    def any(self) -> bool:
        return self.on

    @property
    def outer(self) -> bool:
        """The block itself is the region (the layers inside run plainly)."""

        return self.on and self.block

    def expert_chunks(self, rows: int) -> list[tuple[int, int]] | None:
        if not self.on or self.block or self.chunks <= 1:
            return None
        step = -(-rows // self.chunks)
        return [(a, min(rows, a + step)) for a in range(0, rows, step)]

    def region(self, level: str, fn, *args):
        """Run ``fn(*args)``, as a recomputed region when this rung of the ladder asks for it."""

        use = self.on and not self.block and (
            (level == "layer" and not self.split and self.chunks <= 1)
            or (level == "half" and (self.split or self.chunks > 1))
            or level == "chunk")
        if not use:
            return fn(*args)
        from torch.utils.checkpoint import checkpoint
        return checkpoint(fn, *args, use_reentrant=False)


def _merge_chunk_aux(parts: list[dict]) -> dict:
    """Routing records of an expert half that ran in row chunks: per-token tensors are concatenated; per-chunk
    dispatch offsets are dropped (the statistics fall back to counting the indices)."""

    out: dict = {}
    for key in parts[0]:
        vals = [p[key] for p in parts]
        if key.endswith("_offsets") or key.endswith("_prob"):
            continue
        if isinstance(vals[0], Tensor):
            out[key] = torch.cat(vals, dim=0)
        elif isinstance(vals[0], dict):
            out[key] = _merge_chunk_aux(vals)
    return out


class Block(nn.Module):
    def __init__(self, s: BlockSpec, init: InitScales, max_sources: int, dense_no_router: bool,
                 depth_reads: bool = True, residual: tuple[str, float] = ("add", 1.0),
                 drop_rates: list[float] | None = None, history_attention: bool = False) -> None:
        super().__init__()
        self.spec = s
        self.depth_reads = depth_reads
        self.history_attention = history_attention
        if history_attention:
            # the block output: one more read over the whole history, then an RMSNorm that restores unit scale (a
            # uniform mixture of M updates has RMS ~ 1/sqrt(M)); reference nestor/backbones/nestor.py:8409-8419
            from nestor_b200.models.scaling import ScaledLinear
            self.out_query = ScaledLinear(s.dim, 1, role="score", bias=False, zero_init=True)
            self.out_key_norm = Norm(s.dim, init.norm_eps)
            self.out_norm = Norm(s.dim, init.norm_eps)
        self.residual = residual       # projection mode: ("add", m) -> x + m*u, ("convex", 1/D) -> (1 - 1/D) x + u/D
        self.group_router = RouterParams(
            s.dim, s.G, s.k, hidden=s.router_hidden, score_lr_mul=s.layers ** -0.5,
            loss_free=s.loss_free, bias_rate=s.bias_rate, noisy=True)
        if s.G == 1:
            self.group_router.requires_grad_(False)
        rates = drop_rates or [0.0] * s.layers
        self.layers = nn.ModuleList([Layer(s, init, max_sources, dense_no_router, depth_reads, rates[i],
                                           bank_experts=s.experts_of_layer(i), history_attention=history_attention)
                                     for i in range(s.layers)])

    def route(self, x: Tensor, noise: Tensor | None, cd: torch.dtype) -> tuple[Tensor, Tensor]:
        """Group router on the block input ``[T, d]`` -> ``(idx [T, k], gates [T, k] fp32)``."""

        s = self.spec
        T = x.shape[0]
        if s.G == 1:
            return (torch.zeros(T, 1, dtype=torch.int64, device=x.device),
                    torch.ones(T, 1, dtype=torch.float32, device=x.device))
        r = self.group_router
        w1, w2 = r.weights("score")
        scores = ops.router_scores(x, W(self, w1), W(self, w2), cd)
        if self.training and r.noise_mlp is not None and not getattr(self, "freeze_routing_noise", False):
            eps = torch.randn_like(scores) if noise is None else noise.to(scores.dtype)
            n1, n2 = r.weights("noise")
            # (an annealing schedule, if any, is already folded into ``noise`` by the backbone: see Nestor.forward)
            scores = scores + eps * torch.nn.functional.softplus(ops.router_scores(x, W(self, n1), W(self, n2), cd))
        if not self.training and not torch.is_grad_enabled():
            self._last_group_prob = torch.softmax(scores.float(), dim=-1).sum(0)
        self.__dict__["_last_scores"] = scores       # reported in the block's aux for the auxiliary losses
        return ops.route_topk(scores, r.choice_bias, s.k, "renorm")

    def forward(self, x: Tensor, sources: list[Tensor], B: int, S: int, cd: torch.dtype,
                pos: Tensor | None, column_mode: bool, noise: Tensor | None = None,
                cache: list | None = None, key_cache: Any = None) -> tuple[list[Tensor], Tensor, dict]:
        """Run the block. ``x [T, d]`` feeds the router; ``sources`` are the completed depth sources its sublayers read
        (one aggregate per earlier block, or every earlier export when the reads are column-resolved). With ``cache``
        (one ``LayerKVCache`` per layer) the rows are one new token per sequence and attention runs against the cache.

        Returns ``(exports, aggregate, aux)``: the depth sources this block contributes (in column mode with
        ``k > 1``: the ``k`` columns, as deviations from their mean if the model re-bases them, then the mean if it is
        exported; a single tensor otherwise), the aggregate (next block's router input), and routing indices.
        """

        s = self.spec
        idx, gates = self.route(x, noise, cd)
        plan = ops.build_column_plan(idx.view(B, S, s.k), s.G, pos) if s.G > 1 and cache is None else None
        ctx = BlockContext(B, S, idx, gates, plan, pos)
        if not self.depth_reads:
            return self._forward_projection(x, ctx, cd, cache, idx)
        if column_mode and s.columns and not s.column_head_only:
            return self._forward_wide_reads(sources, ctx, cd, cache, key_cache, idx)
        streams: Tensor | None = None      # [T, k, d] fp32
        running: Tensor | None = None      # [T, d] fp32 = mean_j streams
        layer_aux = []
        # Merged recurrence (one stream, the gate-weighted sum over a token's columns): every layer of a multi-column
        # block that keeps no per-column streams ('attn_res_kimi', or a block left out of block_column_blocks), and
        # the leading layers of a column block narrowed by block_column_trailing_layers.
        merged_all = s.k > 1 and not (column_mode and s.columns)
        n_merged = len(self.layers) if merged_all else (s.merged_prefix if column_mode else 0)
        prefix: Tensor | None = None
        if n_merged:
            prefix, layer_aux = self._merged_layers(n_merged, sources, ctx, cd, cache, key_cache)
            if merged_all:
                return [prefix], prefix, self._block_aux(idx, layer_aux)
            running = prefix
        rung = RecomputeLadder.current(self.training and cache is None)
        kc = {} if key_cache is None or rung.any else {"key_cache": key_cache}   # scales of the completed sources, shared by all reads
        nsrc = len(sources)

        def attn_half(layer, li, *tensors):
            # tensors = completed sources (+ the running mean from the second layer on): [T, d] each
            n = ops.depth_read_norm(list(tensors), layer.kimi_attn_read.query, layer.kimi_attn_read.value_gains,
                                    layer.attn_norm.weight, layer.kimi_attn_read.eps, layer.attn_norm.eps, cd, **kc)
            return layer.attention(n, ctx, cd) if cache is None else layer.attention_step(n, ctx, cd, cache[li])   # [T, k, d]

        def expert_half(layer, c, *tensors):
            # tensors = completed sources + the mid-layer source, [T, d] each; c = (row begin, row end) or None
            n = ops.depth_read_norm(list(tensors), layer.kimi_mlp_read.query, layer.kimi_mlp_read.value_gains,
                                    layer.mlp_norm.weight, layer.kimi_mlp_read.eps, layer.mlp_norm.eps, cd, **kc)
            return layer.experts(n, ctx if c is None else ctx.rows(*c), cd)

        def one_layer(layer, li, streams, running, *srcs):
            if prefix is None:
                read = list(srcs) if running is None else [*srcs, running]
            else:
                # behind a merged prefix the attention half reads the mean of the tracked window alone, the expert half
                # the whole running aggregate (reference nestor/backbones/nestor.py:7455-7470, 7855-7866)
                read = list(srcs) if streams is None else [*srcs, streams.mean(dim=1)]
            attn = rung.region("half", attn_half, layer, li, *read)
            mid = ops.mid_source(running, attn)
            chunks = rung.expert_chunks(mid.shape[0]) if cache is None else None
            if chunks is None:
                priv, shared, path, aux = rung.region("half", expert_half, layer, None, *srcs, mid)
            else:
                # the expert half over row chunks, each its own region: its activations never exist for all rows at once
                parts = [rung.region("chunk", expert_half, layer, (a, b), *[t[a:b] for t in srcs], mid[a:b])
                         for a, b in chunks]
                priv = None if parts[0][0] is None else torch.cat([p[0] for p in parts], dim=0)
                shared = torch.cat([p[1] for p in parts], dim=0)
                path = None if parts[0][2] is None else torch.cat([p[2] for p in parts], dim=0)
                aux = _merge_chunk_aux([p[3] for p in parts])
            if layer.drop_path > 0.0 and self.training:
                attn = layer.drop(attn, B)
                shared = layer.drop(shared, B)
                priv = None if priv is None else layer.drop(priv, B)
            streams, running = ops.layer_combine(attn, priv, shared, path, streams, running, cd)
            return streams, running, aux

        for li, layer in enumerate(self.layers):
            if li < n_merged:
                continue
            streams, running, aux = rung.region("layer", one_layer, layer, li, streams, running, *sources)
            layer_aux.append(aux)
        assert len(sources) == nsrc
        if column_mode and s.k > 1:
            dev, agg = ops.block_exit(streams)
            if prefix is not None:
                # deviations are re-based on the window's own mean (they still sum to zero); the aggregate carries
                # the merged prefix as well
                agg = prefix + agg
            exports = [*(dev.unbind(dim=0) if s.column_deviation else streams.unbind(dim=1)), agg]
        else:
            agg = streams.mean(dim=1) if s.k > 1 else streams[:, 0]
            exports = [agg]
            if prefix is not None:
                # a single-column block exports its tracked window; the next block's router sees prefix + window
                # (reference nestor/backbones/nestor.py:9466-9474)
                agg = prefix + agg
        return exports, agg, self._block_aux(idx, layer_aux)

    def _live_sources(self, streams: Tensor) -> list[Tensor]:
        """This block's entries of a column-resolved read / its exports: the ``k`` streams (as deviations from their
        mean if the model re-bases them), then the mean if it is exported; a single-column block is its one stream
        (reference ``nestor/backbones/nestor.py:860-909``)."""

        s = self.spec
        if s.k == 1:
            return [streams[:, 0]]
        agg = streams.mean(dim=1)
        cols = streams - agg.unsqueeze(1) if s.column_deviation else streams
        return [*cols.unbind(dim=1), *([agg] if s.column_aggregate else [])]

    def _forward_wide_reads(self, sources: list[Tensor], ctx: "BlockContext", cd: torch.dtype, cache: list | None,
                            key_cache: Any, idx: Tensor) -> tuple[list[Tensor], Tensor, dict]:
        """Column mode whose sublayer reads are column-resolved (``block_column_head_only=False``): ``sources`` holds
        every export of the completed blocks, and each read appends this block's live streams to them
        (reference ``nestor/backbones/nestor.py:7172-7254``, ``7301-7318``). A merged prefix
        (``block_column_trailing_layers``) only enters the aggregate handed to the next block's router. Under the
        recompute ladder every layer is one region (the rungs that split a layer fall back to that)."""

        s = self.spec
        rung = RecomputeLadder.current(self.training and cache is None)
        kc = {} if key_cache is None or rung.any else {"key_cache": key_cache}
        layer_aux: list = []
        prefix: Tensor | None = None
        n_merged = s.merged_prefix
        if n_merged:
            prefix, layer_aux = self._merged_layers(n_merged, sources, ctx, cd, cache, key_cache)

        def one_layer(layer, li, streams, running, *srcs):
            read = list(srcs) if streams is None else [*srcs, *self._live_sources(streams)]
            n = ops.depth_read_norm(read, layer.kimi_attn_read.query, layer.kimi_attn_read.value_gains,
                                    layer.attn_norm.weight, layer.kimi_attn_read.eps, layer.attn_norm.eps, cd, **kc)
            attn = layer.attention(n, ctx, cd) if cache is None else layer.attention_step(n, ctx, cd, cache[li])
            if layer.drop_path > 0.0 and self.training:
                attn = layer.drop(attn, ctx.B)
            mid = attn.float() if streams is None else streams + attn.float()
            n = ops.depth_read_norm([*srcs, *self._live_sources(mid)], layer.kimi_mlp_read.query,
                                    layer.kimi_mlp_read.value_gains, layer.mlp_norm.weight, layer.kimi_mlp_read.eps,
                                    layer.mlp_norm.eps, cd, **kc)
            priv, shared, path, aux = layer.experts(n, ctx, cd)
            if layer.drop_path > 0.0 and self.training:
                shared = layer.drop(shared, ctx.B)
                priv = None if priv is None else layer.drop(priv, ctx.B)
            streams, running = ops.layer_combine(attn, priv, shared, path, streams, running, cd)
            return streams, running, aux

        streams: Tensor | None = None
        running: Tensor | None = None
        for li, layer in enumerate(self.layers):
            if li < n_merged:
                continue
            # every rung but the block-level one makes the layer a recomputed region here (no split halves)
            if rung.on and not rung.block:
                from torch.utils.checkpoint import checkpoint
                streams, running, aux = checkpoint(one_layer, layer, li, streams, running, *sources, use_reentrant=False)
            else:
                streams, running, aux = one_layer(layer, li, streams, running, *sources)
            layer_aux.append(aux)
        exports = self._live_sources(streams)
        agg = exports[-1] if (s.k == 1 or s.column_aggregate) else streams.mean(dim=1)
        if prefix is not None:
            agg = prefix + agg
            if s.k > 1 and s.column_aggregate:
                exports[-1] = agg
        return exports, agg, self._block_aux(idx, layer_aux)

    def _block_aux(self, idx: Tensor, layer_aux: list) -> dict:
        s = self.spec
        baux = {"group_idx": idx, "layers": layer_aux}
        scores = self.__dict__.pop("_last_scores", None)
        if s.G > 1 and scores is not None:
            # what the auxiliary losses read (reference aux layout, tokens flattened): raw scores incl. training noise
            baux["group_router"] = {"scores": scores, "topk_indices": idx}
        if not self.training and not torch.is_grad_enabled() and s.G > 1:
            baux["group_prob"] = self.__dict__.pop("_last_group_prob", None)
        return baux

    @staticmethod
    def _merged_expert_update(priv: Tensor | None, shared: Tensor, path: Tensor | None, cd: torch.dtype) -> Tensor:
        """One ``[T, d]`` fp32 update from an expert half: path-weighted public + path-weighted sum of the private slots
        (weights absent for banks, dense layers and the private-only pool)."""

        if path is not None:
            update = (path[:, 0:1].float() * shared.float()).to(cd).float()
            if priv is not None:
                update = update + (path[:, 1:2].float() * priv.float().sum(dim=1)).to(cd).float()
            return update
        update = shared.float()
        return update if priv is None else update + priv.float().sum(dim=1)

    def _merged_layers(self, count: int, sources: list[Tensor], ctx: "BlockContext", cd: torch.dtype,
                       cache: list | None, key_cache: Any) -> tuple[Tensor, list]:
        """The first ``count`` layers as the merged recurrence: every sublayer reads the completed sources plus the
        running sum ``partial`` of this block's updates, and adds its update, summed over the token's columns, to it
        (reference ``nestor/backbones/nestor.py:7005-7034``). Returns ``(partial [T, d] fp32, per-layer aux)``."""

        rung = RecomputeLadder.current(self.training and cache is None)
        kc = {} if key_cache is None or rung.any else {"key_cache": key_cache}

        def attn_part(layer, li, *tensors):
            # tensors = completed sources (+ the partial sum from the second sublayer on)
            n = ops.depth_read_norm(list(tensors), layer.kimi_attn_read.query, layer.kimi_attn_read.value_gains,
                                    layer.attn_norm.weight, layer.kimi_attn_read.eps, layer.attn_norm.eps, cd, **kc)
            attn = layer.attention(n, ctx, cd) if cache is None else layer.attention_step(n, ctx, cd, cache[li])
            return layer.drop(attn.float().sum(dim=1), ctx.B)

        def expert_part(layer, *tensors):
            # tensors = completed sources + the partial sum
            n = ops.depth_read_norm(list(tensors), layer.kimi_mlp_read.query, layer.kimi_mlp_read.value_gains,
                                    layer.mlp_norm.weight, layer.kimi_mlp_read.eps, layer.mlp_norm.eps, cd, **kc)
            priv, shared, path, aux = layer.experts(n, ctx, cd)
            return layer.drop(self._merged_expert_update(priv, shared, path, cd), ctx.B), aux

        def one_layer(layer, li, partial, *srcs):
            read = srcs if partial is None else (*srcs, partial)
            update = rung.region("half", attn_part, layer, li, *read)
            partial = update if partial is None else partial + update
            update, aux = rung.region("half", expert_part, layer, *srcs, partial)
            return partial + update, aux

        partial: Tensor | None = None
        layer_aux = []
        for li, layer in enumerate(self.layers[:count]):
            # the same rungs as the column layers: a layer, or each of its halves, is a recomputed region
            partial, aux = rung.region("layer", one_layer, layer, li, partial, *sources)
            layer_aux.append(aux)
        return partial, layer_aux


    def _apply_residual(self, x: Tensor, update: Tensor) -> Tensor:
        rule, c = self.residual
        return x + c * update if rule == "add" else (1.0 - c) * x + c * update

    def _forward_projection(self, x: Tensor, ctx: "BlockContext", cd: torch.dtype, cache: list | None,
                            idx: Tensor) -> tuple[list[Tensor], Tensor, dict]:
        """Plain pre-norm residual block (``block_residual_mode='projection'``): every layer adds its attention and
        expert updates to one fp32 stream with the model's residual rule, a token's update being the gate-weighted
        sum over its columns (reference ``nestor/backbones/nestor.py:4746-4763``, ``:4918-4940``)."""

        if self.history_attention:
            return self._forward_history_attention(x, ctx, cd, cache, idx)
        layer_aux = []
        for li, layer in enumerate(self.layers):
            n = ops.stream_rmsnorm(x, layer.attn_norm.weight, layer.attn_norm.eps, cd)
            attn = layer.attention(n, ctx, cd) if cache is None else layer.attention_step(n, ctx, cd, cache[li])
            x = self._apply_residual(x, layer.drop(attn.float().sum(dim=1), ctx.B))
            n = ops.stream_rmsnorm(x, layer.mlp_norm.weight, layer.mlp_norm.eps, cd)
            priv, shared, path, aux = layer.experts(n, ctx, cd)
            x = self._apply_residual(x, layer.drop(self._merged_expert_update(priv, shared, path, cd), ctx.B))
            layer_aux.append(aux)
        baux = {"group_idx": idx, "layers": layer_aux}
        scores = self.__dict__.pop("_last_scores", None)
        if self.spec.G > 1 and scores is not None:
            baux["group_router"] = {"scores": scores, "topk_indices": idx}
        return [x], x, baux


    def _forward_history_attention(self, x: Tensor, ctx: "BlockContext", cd: torch.dtype, cache: list | None,
                                   idx: Tensor) -> tuple[list[Tensor], Tensor, dict]:
        """``residual_mode='attn_res'``: no residual stream inside the block. The history starts with the block input;
        every sublayer reads a softmax mixture of the whole history, normalises it, and appends its update (summed
        over the token's columns); the block output is one more read over the history followed by ``out_norm``
        (reference ``nestor/backbones/nestor.py:6913-6950``, ``9547-9572``)."""

        # (the history's inverse RMS uses the op's own 1e-6 floor, not the key norms' epsilon: the reference caches it
        # with that default, nestor/backbones/nestor.py:3900-3914)
        history = [x]
        layer_aux = []
        for li, layer in enumerate(self.layers):
            h = ops.depth_attention(history, layer.attn_query.weight, layer.attn_key_norm.weight)
            n = ops.stream_rmsnorm(h, layer.attn_norm.weight, layer.attn_norm.eps, cd)
            attn = layer.attention(n, ctx, cd) if cache is None else layer.attention_step(n, ctx, cd, cache[li])
            history.append(layer.drop(attn.float().sum(dim=1), ctx.B))
            h = ops.depth_attention(history, layer.mlp_query.weight, layer.mlp_key_norm.weight)
            n = ops.stream_rmsnorm(h, layer.mlp_norm.weight, layer.mlp_norm.eps, cd)
            priv, shared, path, aux = layer.experts(n, ctx, cd)
            history.append(layer.drop(self._merged_expert_update(priv, shared, path, cd), ctx.B))
            layer_aux.append(aux)
        out = ops.depth_attention(history, self.out_query.weight, self.out_key_norm.weight)
        out = ops.stream_rmsnorm(out, self.out_norm.weight, self.out_norm.eps, torch.float32)
        baux = {"group_idx": idx, "layers": layer_aux}
        scores = self.__dict__.pop("_last_scores", None)
        if self.spec.G > 1 and scores is not None:
            baux["group_router"] = {"scores": scores, "topk_indices": idx}
        return [out], out, baux


class Nestor(Backbone):
    """The backbone: blocks, the final head read over every export, the final RMSNorm."""

    def __init__(self, config: NestorConfig, mup: ReferenceMupConfig | None = None,
                 dense_no_router: bool = True) -> None:
        super().__init__()
        self.config = config
        self.specs = config.resolve()
        self.column_mode = config.column_mode
        # column mode with column-resolved sublayer reads: blocks read every export so far, not one aggregate per block
        self.wide_reads = config.column_mode and not config.block_column_head_only
        self.max_depth_sources = config.max_depth_sources()
        total_layers = sum(s.layers for s in self.specs)
        init = InitScales(mup, config.input_dim, total_layers)
        self.depth_reads = config.depth_reads
        # projection mode: additive rule with the reference-muP multiplier, else the convex rule with 1/D, D = 2 * layers
        residual = ("add", mup.residual_multiplier) if mup is not None else ("convex", 1.0 / (2 * total_layers))
        # stochastic depth rises linearly over the layers of a block (timm rule): 0 for its first layer, the
        # configured rate for its last (reference ``nestor/backbones/nestor.py:2338-2345``)
        rates = [[config.drop_path_rate * i / max(s.layers - 1, 1) for i in range(s.layers)] for s in self.specs]
        self.blocks = nn.ModuleList(
            [Block(s, init, self.max_depth_sources, dense_no_router, self.depth_reads, residual, rates[i],
                   history_attention=config.history_attention)
             for i, s in enumerate(self.specs)])
        if self.depth_reads:
            self.final_depth_read = DepthRead(config.output_dim, self.max_depth_sources,
                                              per_source_queries=config.block_column_head_query_per_source)
        # 'attn_res': plain residual blocks joined by a per-source key/value mixture of the block outputs so far
        self.block_attention_residuals: nn.ModuleList | None = None
        if config.block_residual_mode == "attn_res":
            d, emb = config.input_dim, int(config.block_attn_res_include_embedding)
            self.block_attention_residuals = nn.ModuleList(
                [BlockAttentionResidual([d] * (b + 1 + emb), d, std=1.0 / math.sqrt(d)) for b in range(len(self.specs))])
        self.final_norm = Norm(config.output_dim, init.norm_eps)
        lam = config.block_column_mass_lambda
        if self.depth_reads and self.column_mode and (config.block_column_gain_init != 1.0 or lam is not None):
            # Head-read gains: deviation slots of every multi-column block start at the configured value (0 for the
            # registered cells); embedding, aggregates and merged blocks stay 1. With block_column_mass_lambda each
            # multi-column block holds one unit of init mass instead: lambda / k per column, 1 - lambda on the
            # aggregate (reference nestor/backbones/nestor.py:10106-10145).
            g = torch.ones(self.max_depth_sources)
            slot = 1
            for s in self.specs:
                if s.k > 1 and s.columns:
                    g[slot : slot + s.k] = config.block_column_gain_init if lam is None else lam / s.k
                    if lam is not None:
                        g[slot + s.k] = 1.0 - lam      # (the aggregate slot exists: resolve() requires it with lambda)
                slot += s.exports
            assert slot == self.max_depth_sources
            # narrow sublayer reads keep their unit init (their slot 1 is an aggregate, not a column); column-resolved
            # sublayer reads share the head read's positional layout, each slicing its prefix
            reads = [self.final_depth_read] if config.block_column_head_only else \
                [m for m in self.modules() if isinstance(m, DepthRead)]
            with torch.no_grad():
                for m in reads:
                    m.value_gains.copy_(g)

    @property
    def output_dim(self) -> int:
        return self.config.output_dim

    def init_kv_cache(self, batch_size: int, max_len: int, device, dtype=torch.float32) -> NestorKVCache:
        """Empty decode state for ``batch_size`` sequences of up to ``max_len`` tokens."""

        return NestorKVCache(self, batch_size, max_len, device, dtype)

    @torch.no_grad()
    def forward_step(self, x0: Tensor, pos: Tensor, cache: NestorKVCache, cd: torch.dtype) -> tuple[Tensor, dict]:
        """One incremental causal step: ``x0 [B, d]`` embeddings of the next token of every sequence at positions
        ``pos [B]`` -> normalised head input ``[B, d]``, with ``cache`` updated in place.

        Depth reads mix a token's own sources over depth, routers and experts act per token, and a column attends
        over the members it has already seen, so feeding a sequence token by token reproduces the full forward
        (in evaluation mode: training noise on the group router is a full-sequence feature). The reference offers
        stepwise decoding for its projection-residual mode only (``nestor/backbones/nestor.py:10442-10506`` raises
        for the depth-read modes the registered models use); this covers those modes.
        """

        if self.training:
            raise RuntimeError("forward_step is an evaluation path: call model.eval() first")
        if not self.config.causal:
            raise RuntimeError("stepwise decoding needs a causal model: a bidirectional token sees later ones")
        B = x0.shape[0]
        with ops.oracle_ops():        # per-token work: the PyTorch statement of the ops on any device
            narrow, wide, x, aux = [x0], [x0], x0, []
            for block, bcache in zip(self.blocks, cache.blocks):
                exports, x, a = block(x, list(wide) if self.wide_reads else narrow, B, 1, cd, pos, self.column_mode, None,
                                      cache=bcache)
                wide.extend(exports)
                narrow = [*narrow, exports[-1]]
                if self.block_attention_residuals is not None:
                    x = self._mix_block_outputs(len(aux), narrow)
                aux.append(a)
            h = self._head_input(wide, narrow, x, cd)
        cache.length += 1
        return h, {"blocks": aux}

    def forward(self, x0: Tensor, B: int, S: int, cd: torch.dtype, pos: Tensor | None = None,
                noises: list[Tensor | None] | None = None) -> tuple[Tensor, dict]:
        """``x0 [T, d]`` fp32 embeddings -> normalised head input ``[T, d]`` in ``cd`` + aux."""

        x0 = ops.grad_sink(x0)   # depth sources are read by every later sublayer: their gradients share a buffer
        narrow = [x0]            # what sublayer reads see: embedding + completed aggregates
        wide = [x0]              # what the head read sees: every export
        x = x0
        aux = []
        # NESTOR_ACTIVATION_CHECKPOINT=1: keep only each block's inputs and recompute its activations in the
        # backward pass (the reference's per-block checkpointing, nestor/train/activation_offload.py:13-35). The
        # recomputation replays the random state, and the kernels are deterministic, so routing repeats exactly.
        rung = RecomputeLadder.current(self.training)
        recompute = rung.any
        noisy = [b.spec.G > 1 and b.group_router.noise_mlp is not None for b in self.blocks]
        anneal = self.training and any(b.group_router.noise_anneal_steps > 0 for b, n in zip(self.blocks, noisy) if n)
        if self.training and (recompute or anneal):
            # Router noise is drawn here, outside every recomputed region, so a region is a pure function of its
            # inputs; an annealing schedule scales the draw here as well and counts this forward once (a replayed region
            # sees the very same tensor again).
            drawn = []
            for i, (b, n) in enumerate(zip(self.blocks, noisy)):
                if not n:
                    drawn.append(None)
                    continue
                eps = torch.randn(x0.shape[0], b.spec.G, device=x0.device) if noises is None or noises[i] is None else noises[i]
                fade = b.group_router.noise_scale(advance=True)
                drawn.append(eps if fade is None else eps * fade.to(eps.dtype))
            noises = drawn
        # Key scales of the completed sources are shared by every sublayer read (NESTOR_NO_DEPTH_KEY_CACHE=1 turns the
        # sharing off). Off under recomputation, as in the reference (nestor/backbones/nestor.py:10334-10346): a replayed
        # block must not pick up tensors of the first pass. The fused kernel ignores it (the scale is free there).
        key_cache = None
        if (self.depth_reads and not recompute and not ops.use_kernels(x0)
                and os.environ.get("NESTOR_NO_DEPTH_KEY_CACHE") != "1"):
            key_cache = ops.DepthKeyCache(wide if self.wide_reads else narrow, eps=self.final_depth_read.eps)
        self.last_key_cache = key_cache
        for i, block in enumerate(self.blocks):
            noise = None if noises is None else noises[i]
            reads = list(wide) if self.wide_reads else narrow     # (a snapshot: ``wide`` grows in place below)
            if rung.outer:
                from torch.utils.checkpoint import checkpoint
                exports, x, a = checkpoint(block, x, reads, B, S, cd, pos, self.column_mode, noise, use_reentrant=False)
            else:
                exports, x, a = block(x, reads, B, S, cd, pos, self.column_mode, noise, key_cache=key_cache)
            same = x is exports[-1]
            exports = [ops.grad_sink(e) for e in exports]
            if same:
                x = exports[-1]      # the aggregate is the block's last export
            wide.extend(exports)
            narrow = [*narrow, exports[-1]]
            if key_cache is not None:
                key_cache.extend(exports if self.wide_reads else [exports[-1]])
            if self.block_attention_residuals is not None:
                x = self._mix_block_outputs(i, narrow)
            aux.append(a)
        return self._head_input(wide, narrow, x, cd), {"blocks": aux}

    def _mix_block_outputs(self, block_index: int, narrow: list[Tensor]) -> Tensor:
        """Input of the next block in 'attn_res' mode: the mixture of the embedding (optional) and the block outputs."""

        srcs = narrow if self.config.block_attn_res_include_embedding else narrow[1:]
        return self.block_attention_residuals[block_index](srcs)

    def _head_input(self, wide: list[Tensor], narrow: list[Tensor], x: Tensor, cd: torch.dtype) -> Tensor:
        """The normalised head input: the final depth read over every export, or (projection mode) the stream itself."""

        if not self.depth_reads:
            return ops.stream_rmsnorm(x, self.final_norm.weight, self.final_norm.eps, cd)
        read_sources = wide if self.column_mode else narrow
        return ops.depth_read_norm(read_sources, self.final_depth_read.query, self.final_depth_read.value_gains,
                                   self.final_norm.weight, self.final_depth_read.eps, self.final_norm.eps, cd)

    def routers(self) -> list[tuple[str, RouterParams]]:
        return [(n, m) for n, m in self.named_modules() if isinstance(m, RouterParams)]


# ------------------------------------------------------------------ loss-free balancing


def _count(idx: Tensor, n: int, valid: Tensor | None = None) -> Tensor:
    """Histogram of ``idx [T, ...]`` over ``n`` bins without a host sync; ``valid [T]`` drops padding tokens."""

    flat = idx.reshape(-1).long()
    if valid is None:
        w = torch.ones_like(flat, dtype=torch.float32)
    else:
        w = valid.reshape(-1, *([1] * (idx.dim() - 1))).expand_as(idx).reshape(-1).to(torch.float32)
    return torch.zeros(n, dtype=torch.float32, device=idx.device).scatter_add_(0, flat, w)


class RouterCounts(dict):
    """Selection counts of every router, keyed by module path, whose values are views of one flat fp32 tensor.

    A model has some two hundred routers; summing their counts over the micro-batches of a step key by key costs as
    many tiny launches per micro-batch. ``total.add_(counts)`` is one.
    """

    flat: Tensor

    @classmethod
    def pack(cls, counts: dict[str, Tensor]) -> "RouterCounts":
        out = cls()
        names = sorted(counts)
        if not names:
            out.flat, out.layout = torch.zeros(0), []
            return out
        out.flat = torch.cat([counts[n].reshape(-1).float() for n in names])
        out._wire(names, [counts[n].shape for n in names])
        return out

    def _wire(self, names, shapes) -> None:
        off = 0
        self.layout = list(zip(names, shapes))
        for n, shape in self.layout:
            size = int(torch.Size(shape).numel())
            self[n] = self.flat[off : off + size].view(shape)
            off += size

    def clone(self) -> "RouterCounts":
        out = RouterCounts()
        out.flat = self.flat.clone()
        out._wire([n for n, _ in self.layout], [s for _, s in self.layout])
        return out

    def add_(self, other: "RouterCounts") -> "RouterCounts":
        self.flat.add_(other.flat)
        return self


def add_router_counts(total: dict | None, counts: dict) -> dict:
    """``total + counts`` for the counts of successive micro-batches (``total`` may be ``None`` or empty)."""

    if isinstance(counts, RouterCounts) and (not total or isinstance(total, RouterCounts)):
        return counts.clone() if not total else total.add_(counts)
    total = {} if total is None else total
    for k, v in counts.items():
        total[k] = v if k not in total else total[k] + v
    return total


@torch.no_grad()
def router_counts(backbone: Nestor, aux: dict) -> dict[str, Tensor]:
    """Per-router selection counts of one forward, keyed by the router's module path.

    Private routers count only tokens routed into their column (the reference passes each
    private router the mask ``valid & member``, ``expert_pools.py:533-586``).
    """

    out: dict[str, Tensor] = {}
    valid = aux.get("valid_token_mask")
    valid = None if valid is None else valid.reshape(-1)
    for b, (block, baux) in enumerate(zip(backbone.blocks, aux["blocks"])):
        s = block.spec
        if s.G > 1:
            out[f"blocks.{b}.group_router"] = _count(baux["group_idx"], s.G, valid)
        for l, (layer, laux) in enumerate(zip(block.layers, baux["layers"])):
            base = f"blocks.{b}.layers.{l}"
            if layer.expert_pool is not None:
                has_public = layer.expert_pool.has_public
                if "private_offsets" in laux and valid is None:     # the dispatch plans already hold the per-expert histograms
                    if has_public:
                        out[f"{base}.expert_pool.public_router"] = laux["public_offsets"].diff().float()
                    per = laux["private_offsets"].diff().float().view(s.G, s.Q)
                else:
                    if has_public:
                        out[f"{base}.expert_pool.public_router"] = _count(laux["public_idx"], s.P, valid)
                    flat = laux["columns"].long().unsqueeze(-1) * s.Q + laux["private_idx"].long()
                    per = _count(flat, s.G * s.Q, valid).view(s.G, s.Q)
                for g in range(s.G):
                    out[f"{base}.expert_pool.private_routers.{g}"] = per[g]
            elif "expert_idx" in laux:
                out[f"{base}.expert_router"] = _count(laux["expert_idx"], layer.bank_experts, valid)
    return out


def router_prob_sums(backbone: Nestor, aux: dict) -> dict[str, Tensor]:
    """Summed softmax routing probabilities of one evaluation forward, keyed like :func:`router_counts`
    (present only for forwards run in eval mode without gradients)."""

    out: dict[str, Tensor] = {}
    for b, (block, baux) in enumerate(zip(backbone.blocks, aux["blocks"])):
        s = block.spec
        if baux.get("group_prob") is not None:
            out[f"blocks.{b}.group_router"] = baux["group_prob"]
        for l, (layer, laux) in enumerate(zip(block.layers, baux["layers"])):
            base = f"blocks.{b}.layers.{l}"
            if "private_prob" in laux:
                if "public_prob" in laux:
                    out[f"{base}.expert_pool.public_router"] = laux["public_prob"]
                for g in range(s.G):
                    out[f"{base}.expert_pool.private_routers.{g}"] = laux["private_prob"][g]
            elif "expert_prob" in laux:
                out[f"{base}.expert_router"] = laux["expert_prob"]
    return out


@torch.no_grad()
def apply_bias_updates(backbone: Nestor, counts: dict[str, Tensor], *, global_counts: bool = False) -> None:
    """Loss-free balancing nudge after an optimizer step: ``bias += rate * sign(mean(c) - c)``.

    ``counts`` holds the window's summed selection counts per router (reference
    ``nestor.py:596-634``). ``global_counts`` sums them over ranks first, which makes every
    rank compute the same update (the ``NESTOR_LOSSFREE_GLOBAL_COUNTS`` behaviour) — all
    routers travel in one packed all-reduce.
    """

    if not counts:
        return
    names = sorted(counts)
    multi = global_counts and torch.distributed.is_available() and torch.distributed.is_initialized() \
        and torch.distributed.get_world_size() > 1
    if isinstance(counts, RouterCounts) and counts.flat.is_cuda and counts.flat.numel() > 0:
        # packed counts on a GPU: one all-reduce of the flat tensor (if asked for) and one kernel for every router
        if multi:
            torch.distributed.all_reduce(counts.flat)
        _fused_bias_update(backbone, counts)
        return
    if multi:
        flat = torch.cat([counts[n].reshape(-1) for n in names])
        torch.distributed.all_reduce(flat)
        off = 0
        for n in names:
            k = counts[n].numel()
            counts[n] = flat[off : off + k]
            off += k
    modules = dict(backbone.named_modules())
    for n in names:
        r = modules[n]
        if r.loss_free and r.bias_rate:
            c = counts[n]
            r.choice_bias.add_(r.bias_rate * torch.sign(c.mean() - c))


def _fused_bias_update(backbone: Nestor, counts: RouterCounts) -> None:
    """``nb_bias_update``: the table of (bias pointer, offset into the flat counts, size, rate) is built once per
    backbone and layout (router buffers do not move), the flat counts pointer is a launch argument."""

    import ctypes as C

    from nestor_b200.ops import _lib
    names = [n for n, _ in counts.layout]
    cache = backbone.__dict__.setdefault("_bias_update_tables", {})
    key = (tuple(names), counts.flat.device)
    hit = cache.get(key)
    if hit is not None and [r.choice_bias.data_ptr() for r in hit[3]] != hit[2]:
        hit = None                                   # a buffer was re-created (model moved or rebuilt): new table
    if hit is None:
        modules = dict(backbone.named_modules())
        rows, off = [], 0
        for n, shape in counts.layout:
            size = int(torch.Size(shape).numel())
            r = modules[n]
            if r.loss_free and r.bias_rate:
                assert r.choice_bias.numel() == size and r.choice_bias.dtype == torch.float32 and r.choice_bias.is_contiguous()
                rate = torch.tensor([r.bias_rate], dtype=torch.float32).view(torch.int32).item()
                rows.append([r.choice_bias.data_ptr(), off, size | (rate << 32)])
            off += size
        table = torch.tensor(rows, dtype=torch.int64).reshape(-1, 3).to(counts.flat.device) if rows else None
        routers = [modules[n] for n in names]
        hit = cache[key] = (table, len(rows), [r.choice_bias.data_ptr() for r in routers], routers)
    table, n_rows = hit[0], hit[1]
    if n_rows == 0:
        return
    L = _lib.lib()
    L.nb_bias_update.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]
    L.nb_bias_update.restype = C.c_int
    rc = L.nb_bias_update(table.data_ptr(), n_rows, counts.flat.data_ptr(), C.c_void_p(_lib.stream_ptr()))
    if rc != 0:
        raise RuntimeError(f"nb_bias_update failed with code {rc}")
    _lib.count_launch()
