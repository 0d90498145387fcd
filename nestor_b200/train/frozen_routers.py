"""Freeze every routing decision of a model (domain adaptation with fixed routing).

``freeze_routers(model)`` turns off gradients for every router's score / noise matrices and the
pool path gates stay trainable (they mix, they do not route); loss-free balancing biases stop
moving (``bias_rate = 0``); the exploration noise of the group routers is disabled by holding the
routers in eval mode (``hold_routing_in_eval_mode``) so training and evaluation route identically.
Recognition is structural (any ``RouterParams`` module), like the reference's
``nestor/train/frozen_routers.py:81-189``.
"""

from __future__ import annotations

from torch import nn

from nestor_b200.models.modules import RouterParams


def router_modules(model: nn.Module) -> list[tuple[str, RouterParams]]:
    return [(n, m) for n, m in model.named_modules() if isinstance(m, RouterParams)]


def freeze_routers(model: nn.Module) -> int:
    """Freeze all routers; returns the number of parameter tensors frozen."""

    frozen = 0
    for _, r in router_modules(model):
        for p in r.parameters():
            if p.requires_grad:
                p.requires_grad_(False)
                frozen += 1
        r.bias_rate = 0.0
        r.loss_free = False
    hold_routing_in_eval_mode(model)
    return frozen


def hold_routing_in_eval_mode(model: nn.Module) -> None:
    """Make ``model.train()`` leave the blocks' group routers deterministic (no exploration noise)."""

    for m in model.modules():
        if hasattr(m, "group_router") and isinstance(m.group_router, RouterParams):
            m.freeze_routing_noise = True


def routers_are_frozen(model: nn.Module) -> bool:
    return all(not p.requires_grad for _, r in router_modules(model) for p in r.parameters())
