"""Per-parameter optimizer tags.

Every trainable tensor carries a :class:`ParamTag` naming its optimizer (``"muon"`` or
``"adamw"``), learning-rate multiplier, Muon spectral scale ``sqrt(d_out / d_in)`` and
whether decoupled weight decay applies. The optimizer builder groups parameters by
these tags. Same contract as the reference's ``ParamScaling`` (``nestor/scaling/blocks.py:45-96``).
"""

from __future__ import annotations

import dataclasses as dc
import math

import torch
from torch import nn

_ATTR = "_nestor_tag"


@dc.dataclass(frozen=True)
class ParamTag:
    optimizer: str
    lr_mul: float = 1.0
    muon_scale: float = 1.0
    weight_decay: bool = True


def tag(param: nn.Parameter, t: ParamTag) -> nn.Parameter:
    setattr(param, _ATTR, t)
    return param


def get_tag(param: object) -> ParamTag | None:
    t = getattr(param, _ATTR, None)
    return t if isinstance(t, ParamTag) else None


def muon_matrix(d_out: int, d_in: int) -> ParamTag:
    """Tag of an in-stream matrix mapping ``d_in -> d_out``."""

    return ParamTag("muon", muon_scale=math.sqrt(d_out / d_in))


ADAMW_DECAY = ParamTag("adamw", lr_mul=1.0, weight_decay=True)
ADAMW_NO_DECAY = ParamTag("adamw", lr_mul=1.0, weight_decay=False)


def copy_tags(dst: nn.Module, src: nn.Module) -> None:
    """Carry tags across a structural copy (tags live on tensors, not in ``state_dict``)."""

    src_params = dict(src.named_parameters())
    for name, p in dst.named_parameters():
        t = get_tag(src_params.get(name))
        if t is not None:
            tag(p, t)


def zeros_param(*shape: int) -> nn.Parameter:
    return nn.Parameter(torch.zeros(*shape))
