"""Checkpoint save / load in the reference's on-disk format.

A checkpoint is ``torch.save`` of ``{"model": fp32 state_dict with unwrapped key names,
"step", "epoch", "git_sha", "optimizer": unsharded torch-format state, "scheduler",
["config"], ["metrics"], ["ema"]}`` (reference ``nestor/train/checkpoint.py:180-253``).
Loading is strict for resume; initialisation from another run's file is by name and
shape, refuses to leave any *parameter* uncovered unless ``allow_partial`` (``:70-159``),
and applies the legacy key remap ``group_specific_experts.0. -> shared_experts.``
(``:39-67``). Unstacked expert-bank files (per-expert ``layers.0 / layers.1 / gate``
weights) are converted to the stacked layout on load, and can be written back out.
"""

from __future__ import annotations

import re
import subprocess
from pathlib import Path
from typing import Any

import torch
from torch import Tensor, nn

from nestor_b200.utils.distributed import is_main_process

_LEGACY, _CURRENT = "group_specific_experts.0.", "shared_experts."
_BANKS = {
    "expert_pool.public_experts": "expert_pool.stacked_public",
    "expert_pool.private_experts": "expert_pool.stacked_private",
    "shared_experts": "stacked_moe_bank",
}
_PART = {"layers.0.weight": "w_up", "gate.weight": "w_gate", "layers.1.weight": "w_down"}


def get_git_sha() -> str | None:
    try:
        return subprocess.run(["git", "rev-parse", "HEAD"], capture_output=True, text=True, check=True).stdout.strip()
    except (subprocess.CalledProcessError, FileNotFoundError):
        return None


def remap_legacy_bank_keys(state: dict[str, Any], model_keys: set[str]) -> dict[str, Any]:
    out = {}
    for k, v in state.items():
        if _LEGACY in k and k not in model_keys:
            cand = k.replace(_LEGACY, _CURRENT)
            if cand in model_keys:
                k = cand
        out[k] = v
    return out


def is_stacked_state(state: dict[str, Any]) -> bool:
    return any(".stacked_" in k for k in state)


def stack_expert_banks(state: dict[str, Tensor], model_keys: set[str]) -> dict[str, Tensor]:
    """Convert per-expert weights to stacked banks where the model expects stacked keys.

    ``<prefix>.<bank>.{e}.layers.0.weight [h, d]`` (or ``.{g}.{e}.`` for private pools, flat id
    ``g*Q + e``) becomes slice ``e`` of ``<prefix>.<stacked>.w_up [E, d, h]`` (transposed);
    likewise ``gate -> w_gate`` and ``layers.1 -> w_down``.
    """

    pat = re.compile(r"^(.*)\.(expert_pool\.public_experts|expert_pool\.private_experts|shared_experts)"
                     r"\.((?:\d+\.)+)(layers\.0\.weight|layers\.1\.weight|gate\.weight)$")
    found: dict[str, dict[tuple[int, ...], Tensor]] = {}
    out: dict[str, Tensor] = {}
    for k, v in state.items():
        m = pat.match(k)
        if m:
            target = f"{m.group(1)}.{_BANKS[m.group(2)]}.{_PART[m.group(4)]}"
            if target in model_keys and k not in model_keys:
                ids = tuple(int(x) for x in m.group(3).strip(".").split("."))
                found.setdefault(target, {})[ids] = v
                continue
        out[k] = v
    for target, parts in found.items():
        out[target] = torch.stack([parts[i].t() for i in sorted(parts)], dim=0).contiguous()
    return out


def unstack_expert_banks(state: dict[str, Tensor], private_q: dict[str, int] | None = None) -> dict[str, Tensor]:
    """Inverse of :func:`stack_expert_banks` (for exporting to the per-expert layout)."""

    inv = {v: k for k, v in _BANKS.items()}
    part = {v: k for k, v in _PART.items()}
    out: dict[str, Tensor] = {}
    for k, v in state.items():
        m = re.match(r"^(.*)\.(expert_pool\.stacked_public|expert_pool\.stacked_private|stacked_moe_bank)\.(w_up|w_gate|w_down)$", k)
        if not m:
            out[k] = v
            continue
        bank = inv[m.group(2)]
        for e in range(v.shape[0]):
            if bank.endswith("private_experts"):
                q = (private_q or {}).get(m.group(1))
                if q is None:
                    raise ValueError("unstacking a private bank needs Q per layer (private_q).")
                ids = f"{e // q}.{e % q}"
            else:
                ids = str(e)
            out[f"{m.group(1)}.{bank}.{ids}.{part[m.group(3)]}"] = v[e].t().contiguous()
    return out


def filter_init_state(ckpt_state: dict[str, Any], current_state: dict[str, Any], parameter_names: set[str],
                      *, allow_partial: bool = False) -> tuple[dict[str, Any], set[str]]:
    kept = {k: v for k, v in ckpt_state.items()
            if k in current_state and tuple(v.shape) == tuple(current_state[k].shape)}
    skipped = set(ckpt_state) - set(kept)
    uncovered = sorted(parameter_names - set(kept))
    if uncovered and not allow_partial:
        shown = ", ".join(uncovered[:8]) + (" ..." if len(uncovered) > 8 else "")
        raise RuntimeError(
            f"init checkpoint leaves {len(uncovered)} model parameter(s) uninitialised (layout mismatch?): {shown}. "
            "Set DCLM_INIT_ALLOW_PARTIAL=1 only for a deliberately new module.")
    return kept, skipped


def load_init_state(model: nn.Module, ckpt_state: dict[str, Any], *, allow_partial: bool = False) -> tuple[int, set[str]]:
    current = model.state_dict()
    keys = set(current)
    state = stack_expert_banks(remap_legacy_bank_keys(ckpt_state, keys), keys)
    kept, skipped = filter_init_state(state, current, set(dict(model.named_parameters())), allow_partial=allow_partial)
    _load_into(model, kept, strict=False)
    return len(kept), skipped


def _load_into(model: nn.Module, state: dict[str, Tensor], strict: bool) -> None:
    """Copy values into the existing tensors (keeps arena views and tags intact)."""

    current = model.state_dict(keep_vars=True)
    if strict:
        missing, extra = set(current) - set(state), set(state) - set(current)
        if missing or extra:
            raise RuntimeError(f"state dict mismatch: missing {sorted(missing)[:5]}, unexpected {sorted(extra)[:5]}")
    with torch.no_grad():
        for k, v in state.items():
            if k in current:
                if tuple(current[k].shape) != tuple(v.shape):
                    raise RuntimeError(f"shape mismatch for {k}: {tuple(v.shape)} vs {tuple(current[k].shape)}")
                current[k].copy_(v)


def fp32_model_state(model: nn.Module) -> dict[str, Tensor]:
    """Model state with every floating tensor as fp32 on CPU (masters, not compute copies)."""

    out = {}
    for k, v in model.state_dict().items():
        v = v.detach()
        out[k] = (v.float() if v.is_floating_point() else v).cpu().clone()
    return out


def save_checkpoint(path: Path, model: nn.Module, optimizer: Any = None, scheduler: Any = None, *, step: int = 0,
                    epoch: int = 0, config: Any = None, metrics: dict | None = None, ema: dict | None = None) -> None:
    """Collective: every rank calls it (optimizer shards are consolidated), rank 0 writes."""

    if optimizer is not None and hasattr(optimizer, "consolidate_state_dict"):
        optimizer.consolidate_state_dict(to=0)
    if not is_main_process():
        return
    payload: dict[str, Any] = {
        "model": fp32_model_state(model), "step": step, "epoch": epoch, "git_sha": get_git_sha(),
        "optimizer": optimizer.state_dict() if optimizer is not None else None,
        "scheduler": scheduler.state_dict() if scheduler is not None else None,
    }
    if config is not None:
        payload["config"] = config
    if metrics is not None:
        payload["metrics"] = metrics
    if ema is not None:
        payload["ema"] = ema
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    tmp = path.with_suffix(path.suffix + ".tmp")
    torch.save(payload, tmp)
    tmp.replace(path)


def load_checkpoint(path: Path, model: nn.Module, optimizer: Any = None, scheduler: Any = None, *,
                    strict: bool = True, allow_partial: bool = False, map_location: Any = "cpu") -> dict[str, Any]:
    ckpt = torch.load(path, map_location=map_location, weights_only=False)
    state = ckpt["model"] if "model" in ckpt else ckpt
    if strict:
        keys = set(model.state_dict())
        _load_into(model, stack_expert_banks(remap_legacy_bank_keys(state, keys), keys), strict=True)
        if optimizer is not None and ckpt.get("optimizer") is not None:
            optimizer.load_state_dict(ckpt["optimizer"])
        if scheduler is not None and ckpt.get("scheduler") is not None:
            scheduler.load_state_dict(ckpt["scheduler"])
    else:
        load_init_state(model, state, allow_partial=allow_partial)
    return ckpt
