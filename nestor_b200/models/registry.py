"""Config-typed registries of the model parts.

A part (model, adapter, backbone, head) is registered under the config class that describes it; ``build`` looks the
class of a config instance up (walking its MRO, so a subclassed config builds its parent's part) and calls the
registered factory. New parts plug in without touching the composition code:

    @register_backbone(MyBackboneConfig)
    class MyBackbone(Backbone): ...

Same role as the reference's ``register_model / register_adapter / register_head / register_backbone`` decorators and
``*.from_config`` dispatch (``nestor/backbones/base.py:60-91``, ``nestor/models/base.py``).
"""

from __future__ import annotations

import abc
from typing import Any, Callable

from torch import Tensor, nn


class Registry:
    def __init__(self, kind: str) -> None:
        self.kind = kind
        self._factories: dict[type, Callable[..., Any]] = {}

    def register(self, config_type: type) -> Callable:
        def deco(factory: Callable[..., Any]) -> Callable[..., Any]:
            if config_type in self._factories and self._factories[config_type] is not factory:
                raise ValueError(f"a {self.kind} is already registered for {config_type.__name__}")
            self._factories[config_type] = factory
            return factory
        return deco

    def build(self, config: Any, *args: Any, **kwargs: Any) -> Any:
        for klass in type(config).__mro__:
            if klass in self._factories:
                return self._factories[klass](config, *args, **kwargs)
        known = ", ".join(sorted(k.__name__ for k in self._factories)) or "none"
        raise TypeError(f"no {self.kind} registered for {type(config).__name__} (registered: {known})")

    def registered(self) -> dict[type, Callable[..., Any]]:
        return dict(self._factories)


MODELS, ADAPTERS, BACKBONES, HEADS = Registry("model"), Registry("adapter"), Registry("backbone"), Registry("head")
register_model, register_adapter = MODELS.register, ADAPTERS.register
register_backbone, register_head = BACKBONES.register, HEADS.register


class Backbone(nn.Module, abc.ABC):
    """What the sequence model needs from a backbone: flattened tokens in, normalised head input and routing aux out."""

    @property
    @abc.abstractmethod
    def output_dim(self) -> int: ...

    @abc.abstractmethod
    def forward(self, x0: Tensor, B: int, S: int, cd: Any, pos: Tensor | None = None,
                noises: list | None = None) -> tuple[Tensor, dict]: ...
