"""Model composition: text adapter -> Nestor backbone -> language-modelling head."""

from nestor_b200.models.sequence import (  # noqa: F401
    LanguageModelingHead, Model, ModelOutput, SequenceModel, TextAdapter,
)
from nestor_b200.models.nestor import Nestor  # noqa: F401
from nestor_b200.models.registry import (  # noqa: F401
    Backbone, Registry, register_adapter, register_backbone, register_head, register_model,
)
