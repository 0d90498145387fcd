"""Role-typed building blocks: every module carries its own initialisation and optimizer tag.

A weight's *role* decides how it is initialised and which optimizer scaling it gets, so that learning rates transfer
across width and depth without per-model tuning (same contract as the reference's ``nestor/scaling/blocks.py:99-463``):

=============  ==============================================  ===========================================
role           initialisation                                  optimizer tag
=============  ==============================================  ===========================================
``in_stream``  ``N(0, 1/d_in)``                                Muon, spectral scale ``sqrt(d_out/d_in)``
``projection`` semi-orthogonal times ``sqrt(d_out/d_in)``      Muon, spectral scale ``sqrt(d_out/d_in)``
``score``      ``N(0, 1/d_in^2)`` or zeros                     AdamW with ``lr_mul / d_in``
bias / gain    zeros / ones                                    AdamW, no weight decay
embedding      ``N(0, 1)``                                     AdamW at the base rate
=============  ==============================================  ===========================================

These are the general-purpose forms (any leading dimensions, plain PyTorch arithmetic). The backbone's hot path keeps
its parameters in the stacked / arena layouts of :mod:`nestor_b200.models.modules` and runs them through the kernels;
modules outside that path (the block attention residual, custom heads or adapters) are built from the blocks here.
"""

from __future__ import annotations

import math
from typing import Callable

import torch
import torch.nn.functional as F
from torch import Tensor, nn

from nestor_b200.models.tags import ADAMW_DECAY, ADAMW_NO_DECAY, ParamTag, muon_matrix, tag


def _init_in_stream(w: Tensor, d_in: int, d_out: int, zero: bool) -> None:
    nn.init.normal_(w, 0.0, 1.0 / math.sqrt(d_in))


def _init_projection(w: Tensor, d_in: int, d_out: int, zero: bool) -> None:
    nn.init.orthogonal_(w)
    w.mul_(math.sqrt(d_out / d_in))


def _init_score(w: Tensor, d_in: int, d_out: int, zero: bool) -> None:
    if zero:
        nn.init.zeros_(w)
    else:
        nn.init.normal_(w, 0.0, 1.0 / d_in)


ROLES: dict[str, tuple[Callable, Callable[[int, int, float], ParamTag]]] = {
    "in_stream": (_init_in_stream, lambda d_in, d_out, lr_mul: muon_matrix(d_out, d_in)),
    "projection": (_init_projection, lambda d_in, d_out, lr_mul: muon_matrix(d_out, d_in)),
    "score": (_init_score, lambda d_in, d_out, lr_mul: ParamTag("adamw", lr_mul=lr_mul / d_in)),
}


class ScaledLinear(nn.Module):
    """``y = x W^T (+ b)`` with ``W [d_out, d_in]`` initialised and tagged by ``role``.

    ``lr_mul`` multiplies a score head's rate (e.g. ``1/sqrt(M)`` for a router shared by ``M`` layers); ``zero_init``
    starts a score head exactly uniform.
    """

    def __init__(self, in_features: int, out_features: int, *, role: str = "in_stream", bias: bool = True,
                 lr_mul: float = 1.0, zero_init: bool = False) -> None:
        super().__init__()
        if role not in ROLES:
            raise ValueError(f"Unknown role {role!r}. Expected one of {sorted(ROLES)}.")
        self.in_features, self.out_features, self.role = in_features, out_features, role
        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        self.bias = nn.Parameter(torch.zeros(out_features)) if bias else None
        self.reset_parameters(lr_mul=lr_mul, zero_init=zero_init)

    def reset_parameters(self, *, lr_mul: float = 1.0, zero_init: bool = False) -> None:
        init, make_tag = ROLES[self.role]
        with torch.no_grad():
            init(self.weight, self.in_features, self.out_features, zero_init)
            if self.bias is not None:
                self.bias.zero_()
        tag(self.weight, make_tag(self.in_features, self.out_features, lr_mul))
        if self.bias is not None:
            tag(self.bias, ADAMW_NO_DECAY)

    def forward(self, x: Tensor) -> Tensor:
        return F.linear(x, self.weight, self.bias)


_ACTIVATIONS: dict[str, Callable[[Tensor], Tensor]] = {
    "gelu": F.gelu, "relu": F.relu, "silu": F.silu, "tanh": torch.tanh, "identity": lambda x: x,
}


class ScaledMLP(nn.Module):
    """``layers.{i}``: in-stream hidden layers with an activation between them; the last layer takes ``out_role``
    (``"score"`` for routers and prediction heads, ``"in_stream"`` / ``"projection"`` for maps back into the stream)."""

    def __init__(self, in_features: int, hidden_dims: list[int], out_features: int, *, activation: str = "gelu",
                 out_role: str = "in_stream", bias: bool = True, lr_mul: float = 1.0, zero_init: bool = False) -> None:
        super().__init__()
        if activation not in _ACTIVATIONS:
            raise ValueError(f"Unknown activation {activation!r}.")
        dims = [in_features, *hidden_dims, out_features]
        last = len(dims) - 2
        self.layers = nn.ModuleList([
            ScaledLinear(a, b, role=out_role if i == last else "in_stream", bias=bias,
                         lr_mul=lr_mul if i == last else 1.0, zero_init=zero_init and i == last)
            for i, (a, b) in enumerate(zip(dims[:-1], dims[1:]))])
        self.activation = activation

    def forward(self, x: Tensor) -> Tensor:
        act = _ACTIVATIONS[self.activation]
        for layer in self.layers[:-1]:
            x = act(layer(x))
        return self.layers[-1](x)


class GatedScaledMLP(nn.Module):
    """SwiGLU: ``layers.1(silu(gate(x)) * layers.0(x))`` with ``layers = [up, down]`` and a separate ``gate``."""

    gated = True

    def __init__(self, dim: int, hidden: int, *, bias: bool = False) -> None:
        super().__init__()
        self.layers = nn.ModuleList([ScaledLinear(dim, hidden, bias=bias), ScaledLinear(hidden, dim, bias=bias)])
        self.gate = ScaledLinear(dim, hidden, bias=bias)

    def forward(self, x: Tensor) -> Tensor:
        return self.layers[1](F.silu(self.gate(x)) * self.layers[0](x))


class RMSNorm(nn.Module):
    """``x * rsqrt(mean(x^2) + eps) * weight`` with fp32 statistics; ``elementwise_affine=False`` drops the gain."""

    def __init__(self, dim: int, eps: float = 1e-6, elementwise_affine: bool = True) -> None:
        super().__init__()
        self.dim, self.eps = dim, eps
        self.weight = tag(nn.Parameter(torch.ones(dim)), ADAMW_NO_DECAY) if elementwise_affine else None

    def forward(self, x: Tensor) -> Tensor:
        x32 = x.float()
        y = x32 * torch.rsqrt(x32.pow(2).mean(dim=-1, keepdim=True) + self.eps)
        if self.weight is not None:
            y = y * self.weight.float()
        return y.to(x.dtype)


class ScaledEmbedding(nn.Module):
    """Token table with unit-variance rows, AdamW at the base rate (rows are read, never multiplied through)."""

    def __init__(self, num_embeddings: int, dim: int, std: float = 1.0) -> None:
        super().__init__()
        self.weight = tag(nn.Parameter(torch.empty(num_embeddings, dim)), ADAMW_DECAY)
        with torch.no_grad():
            self.weight.normal_(0.0, std)

    def forward(self, ids: Tensor) -> Tensor:
        return F.embedding(ids, self.weight)


class RoPE(nn.Module):
    """Rotate-half rotary embedding in fp32 at integer positions (``head_dim`` even, frequencies ``base^(-2i/d)``)."""

    def __init__(self, head_dim: int, base: float = 10000.0) -> None:
        super().__init__()
        if head_dim % 2:
            raise ValueError("RoPE needs an even head_dim.")
        self.head_dim, self.base = head_dim, float(base)
        self.register_buffer("inv_freq", 1.0 / (self.base ** (torch.arange(0, head_dim, 2).float() / head_dim)),
                             persistent=False)

    def forward(self, x: Tensor, pos: Tensor) -> Tensor:
        """``x [..., S, H, head_dim]`` at positions ``pos [..., S]``."""

        ang = pos.to(torch.float32).unsqueeze(-1) * self.inv_freq
        cos, sin = ang.cos().unsqueeze(-2), ang.sin().unsqueeze(-2)
        x32 = x.float()
        half = self.head_dim // 2
        x1, x2 = x32[..., :half], x32[..., half:]
        return torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin), dim=-1).to(x.dtype)


def convex_residual(h: Tensor, update: Tensor, depth_scale: float) -> Tensor:
    """``(1 - 1/D) h + (1/D) f(h)`` with ``depth_scale = 1/D``, ``D`` the number of residual branches: a convex
    combination keeps the depth-``D`` composition's sensitivity at order one, so no rate carries a depth factor."""

    return (1.0 - depth_scale) * h + depth_scale * update
