"""Parameter-holding building blocks, named so ``state_dict()`` keys match the reference.

Modules here own tensors only; the math lives in :mod:`nestor_b200.ops` so that the
CPU oracle and the sm_100a kernels see the same parameters. All weights are bias-free
(the reference-muP "architecture" component removes every bias,
``nestor/scaling/reference_mup.py:183-203``).

Key layout produced (reference: ``nestor/backbones/expert_bank_stack.py:58-213``,
``nestor/backbones/nestor.py:2979-3010``, ``attention_residual.py:395-480``):

* ``<router>.choice_bias`` (buffer), ``<router>.score_mlp.layers.{i}.weight``,
  ``<router>.noise_mlp.layers.{i}.weight``
* ``attention_groups.{g}.{q,k,v,out}_proj.weight``
* ``stacked_{public,private,moe_bank}.w_{up,gate} [E, d, h]``, ``.w_down [E, h, d]``
* ``shared_experts.0.{layers.0,layers.1,gate}.weight`` for a single dense SwiGLU
* ``kimi_{attn,mlp}_read.{query,value_gains}``
"""

from __future__ import annotations

import math

import torch
from torch import Tensor, nn

from nestor_b200.models.tags import ADAMW_DECAY, ADAMW_NO_DECAY, ParamTag, muon_matrix, tag


class Matrix(nn.Module):
    """A bias-free ``[d_out, d_in]`` weight (``nn.Linear`` layout)."""

    def __init__(self, d_in: int, d_out: int, t: ParamTag, std: float) -> None:
        super().__init__()
        self.in_features, self.out_features = d_in, d_out
        self.weight = tag(nn.Parameter(torch.empty(d_out, d_in)), t)
        self.init_std = std
        self.reset()

    def reset(self) -> None:
        with torch.no_grad():
            if self.init_std == 0.0:
                self.weight.zero_()
            else:
                self.weight.normal_(0.0, self.init_std)


class LayerStack(nn.Module):
    """``layers.{i}.weight`` container (score/noise MLPs, the LM head projection)."""

    def __init__(self, mats: list[Matrix]) -> None:
        super().__init__()
        self.layers = nn.ModuleList(mats)


class Norm(nn.Module):
    """RMSNorm gain (``weight [d]``), AdamW without decay."""

    def __init__(self, dim: int, eps: float) -> None:
        super().__init__()
        self.dim, self.eps = dim, eps
        self.weight = tag(nn.Parameter(torch.ones(dim)), ADAMW_NO_DECAY)


class DepthRead(nn.Module):
    """Pseudo-query ``[d]`` (zero-init) and per-slot value gains ``[max_sources]`` (one-init).

    ``per_source_queries`` gives every slot its own query row (``[max_sources, d]``, still zero-init, so the first
    mixture stays uniform): source ``i`` is scored by ``q_i . k_i`` instead of the shared ``q . k_i``
    (reference ``nestor/backbones/attention_residual.py:448-480``)."""

    def __init__(self, dim: int, max_sources: int, eps: float = 1e-6, per_source_queries: bool = False) -> None:
        super().__init__()
        self.dim, self.max_sources, self.eps = dim, max_sources, eps
        self.per_source_queries = per_source_queries
        self.query = tag(nn.Parameter(torch.zeros(max_sources, dim) if per_source_queries else torch.zeros(dim)),
                         ADAMW_NO_DECAY)
        self.value_gains = tag(nn.Parameter(torch.ones(max_sources)), ADAMW_NO_DECAY)


class RouterParams(nn.Module):
    """Top-k router parameters.

    ``hidden == 0``: the deterministic single-matrix router ``d -> C`` used for every
    pool / bank router under reference muP (``reference_mup.py:51-92``): AdamW at the
    base rate with decay, ``N(0, std^2)``. ``hidden > 0``: the group router's score and
    noise MLPs ``d -> hidden -> C``; the hidden layers are Muon matrices with
    ``N(0, 1/d)`` init, the read-outs AdamW with ``lr_mul = score_lr_mul / hidden`` and
    ``N(0, 1/hidden^2)`` init (``scaling/blocks.py:139-160``). ``choice_bias`` is the
    loss-free balancing buffer.
    """

    def __init__(self, dim: int, choices: int, top_k: int, *, hidden: int = 0, std: float = 0.0,
                 score_lr_mul: float = 1.0, gate_mode: str = "renorm", loss_free: bool = False,
                 bias_rate: float = 0.0, noisy: bool = False) -> None:
        super().__init__()
        self.feature_dim, self.num_choices, self.top_k = dim, choices, top_k
        self.gate_mode, self.loss_free, self.bias_rate = gate_mode, loss_free, bias_rate

        def mlp() -> LayerStack:
            if hidden == 0:
                return LayerStack([Matrix(dim, choices, ADAMW_DECAY, std)])
            return LayerStack([
                Matrix(dim, hidden, muon_matrix(hidden, dim), 1.0 / math.sqrt(dim)),
                Matrix(hidden, choices, ParamTag("adamw", lr_mul=score_lr_mul / hidden), 1.0 / hidden),
            ])

        self.score_mlp = mlp()
        self.noise_mlp = mlp() if noisy else None
        self.register_buffer("choice_bias", torch.zeros(choices))
        # NESTOR_ROUTER_NOISE_ANNEAL_STEPS=n: the exploration noise fades linearly to zero over the first n training
        # forwards; the forward counter is a persistent buffer (it is part of a checkpoint of such a run), reference
        # nestor/backbones/nestor.py:478-484
        import os
        self.noise_anneal_steps = int(os.environ.get("NESTOR_ROUTER_NOISE_ANNEAL_STEPS", "0") or 0) if noisy else 0
        if self.noise_anneal_steps > 0:
            self.register_buffer("_noise_steps", torch.zeros((), dtype=torch.long))

    def noise_scale(self, advance: bool) -> Tensor | None:
        """``1 - min(steps / anneal, 1)`` as a device scalar (``None`` when the noise does not anneal). ``advance``
        counts this forward; recomputed regions and self-checks pass ``False`` so that the schedule follows the
        optimizer's steps, not the number of times a forward is replayed."""

        if self.noise_anneal_steps <= 0:
            return None
        scale = 1.0 - (self._noise_steps.float() / self.noise_anneal_steps).clamp(max=1.0)
        if advance:
            self._noise_steps += 1
        return scale

    def weights(self, which: str = "score") -> tuple[Tensor | None, Tensor]:
        stack = self.score_mlp if which == "score" else self.noise_mlp
        mats = [m.weight for m in stack.layers]
        return (None, mats[0]) if len(mats) == 1 else (mats[0], mats[1])


class ColumnProjections(nn.Module):
    """One attention column: ``{q,k,v}_proj [inner, d]`` and ``out_proj [d, inner]`` (Muon)."""

    def __init__(self, dim: int, inner: int, std: float, out_std: float) -> None:
        super().__init__()
        self.q_proj = Matrix(dim, inner, muon_matrix(inner, dim), std)
        self.k_proj = Matrix(dim, inner, muon_matrix(inner, dim), std)
        self.v_proj = Matrix(dim, inner, muon_matrix(inner, dim), std)
        self.out_proj = Matrix(inner, dim, muon_matrix(dim, inner), out_std)


class ExpertBank(nn.Module):
    """Stacked SwiGLU bank: ``w_up, w_gate [E, d, h]`` and ``w_down [E, h, d]``.

    Each ``[d_in, d_out]`` slice is the transpose of the per-expert ``nn.Linear`` weight the
    unstacked layout stores, so Muon treats the bank as ``E`` independent matrices. ``gated=False`` is the bank of
    pointwise experts ``down(act(up(x)))``: no ``w_gate`` (reference ``nestor/backbones/expert_bank_stack.py:62-130``).
    """

    def __init__(self, experts: int, dim: int, hidden: int, std: float, out_std: float, gated: bool = True) -> None:
        super().__init__()
        self.num_experts, self.dim, self.hidden, self.gated = experts, dim, hidden, gated
        self.w_up = tag(nn.Parameter(torch.empty(experts, dim, hidden)), muon_matrix(hidden, dim))
        self.w_gate = tag(nn.Parameter(torch.empty(experts, dim, hidden)), muon_matrix(hidden, dim)) if gated else None
        self.w_down = tag(nn.Parameter(torch.empty(experts, hidden, dim)), muon_matrix(dim, hidden))
        with torch.no_grad():
            self.w_up.normal_(0.0, std)
            if gated:
                self.w_gate.normal_(0.0, std)
            self.w_down.normal_(0.0, out_std)

    def matrices(self) -> list[nn.Parameter]:
        return [w for w in (self.w_up, self.w_gate, self.w_down) if w is not None]


class DenseExpert(nn.Module):
    """A lone SwiGLU (never stacked): ``layers.0`` = up ``[h, d]``, ``layers.1`` = down ``[d, h]``, ``gate [h, d]``;
    ``gated=False`` is the pointwise MLP ``down(act(up(x)))`` without the gate matrix."""

    def __init__(self, dim: int, hidden: int, std: float, out_std: float, gated: bool = True) -> None:
        super().__init__()
        self.gated = gated
        self.layers = nn.ModuleList([
            Matrix(dim, hidden, muon_matrix(hidden, dim), std),
            Matrix(hidden, dim, muon_matrix(dim, hidden), out_std),
        ])
        self.gate = Matrix(dim, hidden, muon_matrix(hidden, dim), std) if gated else None

    def matrices(self) -> list[Matrix]:
        return [*self.layers, *([self.gate] if self.gate is not None else [])]


class BlockAttentionResidual(nn.Module):
    """Softmax-over-depth mixture of earlier block outputs with per-source key and value projections.

    Source ``i`` (width ``source_widths[i]``) owns ``key_projections.{i}`` and ``value_projections.{i}`` into
    ``target_width``; a zero-initialised query ``[1, target_width]`` scores the projected keys at every position, and
    the output is the convex mixture of the projected values (fp32 softmax across sources). With the query at zero the
    mixture is the plain mean. Used between blocks by ``block_residual_mode='attn_res'``
    (reference ``nestor/backbones/attention_residual.py:259-392``).
    """

    def __init__(self, source_widths: list[int], target_width: int, std: float | None = None) -> None:
        super().__init__()
        if not source_widths or min(source_widths) < 1 or target_width < 1:
            raise ValueError("BlockAttentionResidual needs at least one source and positive widths.")
        self.source_widths, self.target_width = tuple(int(w) for w in source_widths), int(target_width)
        from nestor_b200.models.scaling import ScaledLinear
        mk = lambda w: ScaledLinear(w, target_width, role="projection", bias=False)   # noqa: E731
        self.key_projections = nn.ModuleList([mk(w) for w in self.source_widths])
        self.value_projections = nn.ModuleList([mk(w) for w in self.source_widths])
        self.query = ScaledLinear(target_width, 1, role="score", bias=False, zero_init=True)

    def forward(self, sources: list[Tensor]) -> Tensor:
        if len(sources) != len(self.source_widths):
            raise ValueError(f"Expected {len(self.source_widths)} sources, got {len(sources)}.")
        lead = sources[0].shape[:-1]
        values, logits = [], []
        for i, (src, w, kp, vp) in enumerate(zip(sources, self.source_widths, self.key_projections, self.value_projections)):
            if src.shape[:-1] != lead or src.shape[-1] != w:
                raise ValueError(f"Source {i} must have shape {tuple(lead) + (w,)}, got {tuple(src.shape)}.")
            key = src @ kp.weight.t().to(src.dtype)
            values.append(src @ vp.weight.t().to(src.dtype))
            logits.append((key @ self.query.weight.t().to(src.dtype)).squeeze(-1))
        weights = torch.stack(logits, dim=0).float().softmax(dim=0).to(values[0].dtype)
        return (torch.stack(values, dim=0) * weights.unsqueeze(-1)).sum(dim=0)
