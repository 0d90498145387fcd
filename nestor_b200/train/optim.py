"""Muon + AdamW optimizer (ZeRO-1-style sharded Muon), builders, and LR schedules.

Behaviour reproduced from the reference (``nestor/scaling/muon.py:233-717``,
``nestor/train/optim.py:209-490``):

* Parameters are grouped by their tags: one Muon group per distinct ``round(muon_scale, 8)``
  with ``lr = lr_muon * muon_scale``; one AdamW group per ``(round(lr_mul, 10), decay)``
  with ``lr = lr_adamw * lr_mul``. Groups are emitted in sorted key order, Muon first.
* Muon step: ``buf = mu*buf + g``; Nesterov direction ``g + mu*buf``; quintic Newton–Schulz
  in bf16 on each matrix (stacked ``[E, m, n]`` banks are ``E`` independent matrices, and
  same-shape matrices are orthogonalised in one batched call); decoupled decay
  ``p *= 1 - lr*wd``; ``p -= lr * update``.
* AdamW step: decoupled decay first, then bias-corrected Adam with ``eps`` added after the
  bias-corrected square root.
* Sharding: every Muon parameter has one owner rank, assigned round-robin while walking
  (shape, dtype) buckets in first-seen order. Only the owner keeps momentum and runs
  Newton–Schulz; updated parameters are then distributed to every rank. The distribution
  step is pluggable (``param_sync``) so the fused peer-memory all-gather kernel and the
  plain ``broadcast`` baseline share the optimizer.
"""

from __future__ import annotations

import math
import os
import warnings
from collections import defaultdict
from typing import Any, Callable

import torch
import torch.distributed as dist
from torch import Tensor, nn
from torch.optim import Optimizer
from torch.optim.lr_scheduler import CosineAnnealingLR, LambdaLR, LRScheduler, SequentialLR, StepLR

from nestor_b200 import ops
from nestor_b200.train import fused_optim
from nestor_b200.configs import (
    AdamConfig, AdamWConfig, CosineAnnealingConfig, MuonAdamWConfig, OptimizerConfig, PowerLawConfig,
    SchedulerConfig, SGDConfig, StepLRConfig, WSDConfig,
)
from nestor_b200.models.tags import get_tag


def _fused(*lists: list[Tensor]) -> bool:
    """The multi-tensor kernels apply: CUDA, fp32, contiguous tensors (arena views and their states are)."""

    if os.environ.get("NESTOR_ADAMW_FUSED", "1") != "1":       # the reference's switch between foreach and fused updates
        return False
    return all(t.is_cuda and t.dtype == torch.float32 and t.is_contiguous() for ts in lists for t in ts)


def _dist_on() -> bool:
    return dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1


def orthogonalize(directions: list[Tensor], steps: int) -> list[Tensor]:
    """Newton–Schulz on a list of 2-D matrices / 3-D banks, batched per matrix shape."""

    buckets: dict[tuple, list[int]] = defaultdict(list)
    for i, d in enumerate(directions):
        buckets[(tuple(d.shape[-2:]), d.dtype)].append(i)
    out: list[Tensor | None] = [None] * len(directions)
    for idxs in buckets.values():
        stack = torch.cat([directions[i] if directions[i].ndim == 3 else directions[i].unsqueeze(0)
                           for i in idxs], dim=0)
        # the kernel path hands back bf16 (the iterate's own precision); the parameter update reads it directly
        ortho = ops.newton_schulz(stack, steps, out_dtype=torch.bfloat16 if stack.is_cuda else None)
        counts = [directions[i].shape[0] if directions[i].ndim == 3 else 1 for i in idxs]
        for i, chunk in zip(idxs, ortho.split(counts)):
            out[i] = chunk if directions[i].ndim == 3 else chunk.squeeze(0)
    return out  # type: ignore[return-value]


class MuonAdamW(Optimizer):
    """Muon on ``method == "muon"`` groups, AdamW on the rest; optional owner-sharded Muon."""

    def __init__(self, params: Any, *, lr: float = 1e-3, betas: tuple[float, float] = (0.9, 0.95),
                 eps: float = 1e-8, weight_decay: float = 0.0, momentum: float = 0.95,
                 nesterov: bool = True, ns_steps: int = 5, shard: bool | None = None,
                 param_sync: Callable[["MuonAdamW"], None] | None = None, arena: Any = None) -> None:
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, momentum=momentum,
                        nesterov=nesterov, ns_steps=ns_steps, method="adamw")
        super().__init__(params, defaults)
        if shard is None:
            shard = os.environ.get("NESTOR_MUON_SHARD", "1") == "1"
        self.sharded = bool(shard and _dist_on())
        self.rank = dist.get_rank() if self.sharded else 0
        self.world = dist.get_world_size() if self.sharded else 1
        self.owner: dict[Tensor, int] = {}
        self.owned: list[list[Tensor]] = [[] for _ in range(self.world)]
        self.param_sync = param_sync
        self.arena = arena
        self.owner_cuts: list[int] | None = None   # arena offsets where ownership changes (contiguous mode)
        self._assign_owners()
        # ZeRO-1 for AdamW too (the reference's NESTOR_ZERO1): needs the arena ranges and a parameter distribution step
        # Parameter distribution in arena mode moves whole ownership ranges, AdamW parameters included.
        self.shard_adamw = bool(self.sharded and self.owner_cuts is not None
                                and os.environ.get("NESTOR_ZERO1", "1") == "1")

    # ------------------------------------------------------------------ ownership
    def _assign_owners(self) -> None:
        """Give every Muon parameter one owner rank.

        With a parameter arena the owners hold contiguous arena ranges balanced by element count
        (so the updated parameters of a rank are one range to distribute); without one, owners are
        dealt round-robin over (shape, dtype) buckets in first-seen order, the reference's rule
        (``nestor/scaling/muon.py:319-342``). Which rank updates a matrix does not change the result.
        """

        muon = [p for g in self.param_groups if g.get("method") == "muon" for p in g["params"]]
        if self.arena is not None and muon:
            muon.sort(key=lambda p: self.arena.slot(p).offset)
            total = sum(p.numel() for p in muon)
            cuts, seen = [0], 0
            for p in muon:
                o = min(self.world - 1, seen * self.world // max(total, 1))
                while len(cuts) <= o:
                    cuts.append(self.arena.slot(p).offset)
                self.owner[p] = o
                self.owned[o].append(p)
                seen += p.numel()
            while len(cuts) < self.world:
                cuts.append(self.arena.numel)
            cuts.append(self.arena.numel)
            self.owner_cuts = cuts
            return
        buckets: dict[tuple, list[Tensor]] = defaultdict(list)
        for p in muon:
            buckets[(tuple(p.shape), p.dtype, p.device)].append(p)
        cursor = 0
        for params in buckets.values():
            for p in params:
                o = cursor % self.world
                self.owner[p] = o
                self.owned[o].append(p)
                cursor += 1

    def owned_range(self, rank: int | None = None) -> tuple[int, int]:
        """Arena range ``[lo, hi)`` whose parameters ``rank`` is responsible for distributing."""

        assert self.owner_cuts is not None
        r = self.rank if rank is None else rank
        return self.owner_cuts[r], self.owner_cuts[r + 1]

    def owns(self, p: Tensor) -> bool:
        return (not self.sharded) or self.owner.get(p, self.rank) == self.rank

    def owns_adamw(self, p: Tensor) -> bool:
        """AdamW parameters follow the arena ownership ranges when the optimizer state is fully sharded
        (``shard_adamw``): the owner of a range updates everything in it and distributes the range."""

        if not (self.sharded and self.shard_adamw and self.owner_cuts is not None):
            return True
        off = self.arena.slot(p).offset
        return self.owner_cuts[self.rank] <= off < self.owner_cuts[self.rank + 1]

    # ------------------------------------------------------------------------ step
    @torch.no_grad()
    def step(self, closure: Any = None) -> Any:
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            if group["method"] == "muon":
                self._muon_step(group)
            else:
                self._adamw_step(group)
        if self.sharded:
            (self.param_sync or _broadcast_owned)(self)
        return loss

    def _muon_step(self, group: dict[str, Any]) -> None:
        lr, wd, mu = group["lr"], group["weight_decay"], group["momentum"]
        params, grads, bufs = [], [], []
        for p in group["params"]:
            if not self.owns(p) or p.grad is None:
                continue
            if p.grad.ndim not in (2, 3):
                raise ValueError(f"Muon parameters must be matrices or [E, m, n] banks; got {tuple(p.shape)}.")
            st = self.state[p]
            if "momentum_buffer" not in st:
                st["momentum_buffer"] = torch.zeros_like(p.grad, memory_format=torch.contiguous_format)
            params.append(p)
            grads.append(p.grad)
            bufs.append(st["momentum_buffer"])
        if not params:
            return
        if _fused(params, grads, bufs):
            # one launch for the momentum update of the whole group, one for the parameter update
            directions = [torch.empty_like(b) for b in bufs]
            fused_optim.launch(fused_optim.MOMENTUM, [grads, bufs, directions], [mu, 1.0 if group["nesterov"] else 0.0])
            updates = orthogonalize(directions, group["ns_steps"])
            updates = [u if u.is_contiguous() else u.contiguous() for u in updates]
            op = fused_optim.AXPY_BF16 if updates[0].dtype == torch.bfloat16 else fused_optim.AXPY_F32
            if all(u.dtype == updates[0].dtype and u.dtype in (torch.float32, torch.bfloat16) for u in updates):
                fused_optim.launch(op, [params, updates], [1.0 - lr * wd, -lr])
                return
            if wd != 0.0:
                torch._foreach_mul_(params, 1.0 - lr * wd)
            torch._foreach_add_(params, updates, alpha=-lr)
            return
        torch._foreach_mul_(bufs, mu)
        torch._foreach_add_(bufs, grads)
        directions = torch._foreach_add(grads, bufs, alpha=mu) if group["nesterov"] else bufs
        updates = orthogonalize(list(directions), group["ns_steps"])
        if wd != 0.0:
            torch._foreach_mul_(params, 1.0 - lr * wd)
        torch._foreach_add_(params, updates, alpha=-lr)

    def _adamw_step(self, group: dict[str, Any]) -> None:
        lr, (b1, b2), eps, wd = group["lr"], group["betas"], group["eps"], group["weight_decay"]
        params, grads, m1, m2, steps = [], [], [], [], []
        for p in group["params"]:
            if p.grad is None or not self.owns_adamw(p):
                continue
            st = self.state[p]
            if not st:
                st["step"] = 0
                st["exp_avg"] = torch.zeros_like(p, memory_format=torch.contiguous_format)
                st["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.contiguous_format)
            st["step"] += 1
            params.append(p)
            grads.append(p.grad)
            m1.append(st["exp_avg"])
            m2.append(st["exp_avg_sq"])
            steps.append(st["step"])
        if not params:
            return
        if _fused(params, grads, m1, m2) and len(set(steps)) == 1:
            s = steps[0]
            fused_optim.launch(fused_optim.ADAMW, [params, grads, m1, m2],
                               [1.0 - lr * wd, 1.0 - b1, b2, 1.0 - b2, 1.0 / math.sqrt(1.0 - b2 ** s), eps,
                                lr / (1.0 - b1 ** s)])
            return
        if wd != 0.0:
            torch._foreach_mul_(params, 1.0 - lr * wd)
        torch._foreach_lerp_(m1, grads, 1.0 - b1)
        torch._foreach_mul_(m2, b2)
        torch._foreach_addcmul_(m2, grads, grads, 1.0 - b2)
        denom = torch._foreach_sqrt(m2)
        torch._foreach_div_(denom, [math.sqrt(1.0 - b2 ** s) for s in steps])
        torch._foreach_add_(denom, eps)
        torch._foreach_addcdiv_(params, m1, denom, [-lr / (1.0 - b1 ** s) for s in steps])

    # ------------------------------------------------------------------ state dicts
    @torch.no_grad()
    def consolidate_state_dict(self, to: int = 0) -> None:
        """Bring every owner's momentum to rank ``to`` (call on all ranks before ``state_dict``)."""

        self._consolidated: dict[Tensor, Tensor] = {}
        if not self.sharded:
            return
        for owner in range(self.world):
            for p in self.owned[owner]:
                if owner == self.rank:
                    buf = self.state[p].get("momentum_buffer")
                    buf = torch.zeros_like(p) if buf is None else buf
                else:
                    buf = torch.empty_like(p, memory_format=torch.contiguous_format)
                dist.broadcast(buf, src=owner)
                if self.rank == to and owner != self.rank:
                    self._consolidated[p] = buf
        self._consolidated_adamw: dict[Tensor, dict[str, Any]] = {}
        if self.shard_adamw:
            for g in self.param_groups:
                if g.get("method") == "muon":
                    continue
                for p in g["params"]:
                    off = self.arena.slot(p).offset
                    owner = max(r for r in range(self.world) if self.owner_cuts[r] <= off)
                    st = self.state.get(p, {}) if owner == self.rank else {}
                    step = torch.tensor([float(st.get("step", 0))], device=p.device)
                    dist.broadcast(step, src=owner)
                    bufs = {}
                    for key in ("exp_avg", "exp_avg_sq"):
                        b = st.get(key)
                        b = torch.zeros_like(p, memory_format=torch.contiguous_format) if b is None else b
                        dist.broadcast(b, src=owner)
                        bufs[key] = b
                    if self.rank == to and owner != self.rank and step.item() > 0:
                        self._consolidated_adamw[p] = {"step": int(step.item()), **bufs}

    def state_dict(self) -> dict[str, Any]:
        """Unsharded torch-format state dict (momentum of every Muon parameter present)."""

        extra = getattr(self, "_consolidated", {})
        added = []
        for p, buf in extra.items():
            if "momentum_buffer" not in self.state[p]:
                self.state[p]["momentum_buffer"] = buf
                added.append(p)
        added_adamw = []
        for p, st in getattr(self, "_consolidated_adamw", {}).items():
            if not self.state.get(p):
                self.state[p] = dict(st)
                added_adamw.append(p)
        try:
            return super().state_dict()
        finally:
            for p in added:
                del self.state[p]["momentum_buffer"]
            for p in added_adamw:
                del self.state[p]
            self._consolidated = {}
            self._consolidated_adamw = {}

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        super().load_state_dict(state_dict)
        if self.sharded:  # keep only what this rank owns
            for p, owner in self.owner.items():
                if owner != self.rank and p in self.state:
                    self.state[p].pop("momentum_buffer", None)
            if self.shard_adamw:
                for g in self.param_groups:
                    if g.get("method") != "muon":
                        for p in g["params"]:
                            if not self.owns_adamw(p):
                                self.state.pop(p, None)


@torch.no_grad()
def _broadcast_owned(opt: MuonAdamW) -> None:
    """Baseline parameter distribution: one flat broadcast per owner (reference ``muon.py:410-433``).

    In arena mode an owner's parameters are one contiguous range of the fp32 master buffer, so the range itself is
    broadcast (no flattening copy); it carries the AdamW parameters of the range too.
    """

    if opt.owner_cuts is not None and opt.arena is not None:
        for owner in range(opt.world):
            lo, hi = opt.owned_range(owner)
            if hi > lo:
                dist.broadcast(opt.arena.master[lo:hi], src=owner)
        return
    for owner in range(opt.world):
        ps = opt.owned[owner]
        if not ps:
            continue
        flat = torch.cat([p.detach().reshape(-1) for p in ps])
        dist.broadcast(flat, src=owner)
        if owner != opt.rank:
            off = 0
            for p in ps:
                n = p.numel()
                p.copy_(flat[off : off + n].view_as(p))
                off += n


# ------------------------------------------------------------------------------ builders


def build_param_groups(config: MuonAdamWConfig, model: nn.Module) -> list[dict[str, Any]]:
    muon: dict[float, list[nn.Parameter]] = defaultdict(list)
    adamw: dict[tuple[float, bool], list[nn.Parameter]] = defaultdict(list)
    untagged = []
    # NESTOR_DROP_MUP=1 ignores every tag: one plain AdamW group at the base rate with decay (the regime the reference's
    # first sweeps ran in, ``nestor/train/optim.py:231-238``)
    drop_tags = os.environ.get("NESTOR_DROP_MUP") == "1"
    for name, p in model.named_parameters():
        if not p.requires_grad:
            continue
        t = None if drop_tags else get_tag(p)
        if t is None:
            untagged.append(name)
            adamw[(1.0, True)].append(p)
        elif t.optimizer == "muon":
            muon[round(t.muon_scale, 8)].append(p)
        elif t.optimizer == "adamw":
            adamw[(round(t.lr_mul, 10), t.weight_decay)].append(p)
        else:
            raise ValueError(f"Parameter '{name}' has unknown optimizer '{t.optimizer}'.")
    if untagged and not drop_tags:
        warnings.warn(f"MuonAdamW: {len(untagged)} untagged parameter(s) (e.g. {untagged[0]}) use default AdamW.")
    groups: list[dict[str, Any]] = []
    for scale, ps in sorted(muon.items()):
        groups.append(dict(params=ps, method="muon", lr=config.lr_muon * scale, weight_decay=config.weight_decay,
                           momentum=config.muon_momentum, nesterov=config.muon_nesterov,
                           ns_steps=config.muon_ns_steps))
    for (lr_mul, decay), ps in sorted(adamw.items()):
        groups.append(dict(params=ps, method="adamw", lr=config.lr_adamw * lr_mul, betas=config.betas,
                           eps=config.eps, weight_decay=config.weight_decay if decay else 0.0))
    if not groups:
        raise ValueError("MuonAdamW received a model with no trainable parameters.")
    return groups


def build_optimizer(config: OptimizerConfig, model: nn.Module, **kwargs: Any) -> Optimizer:
    if isinstance(config, MuonAdamWConfig):
        kwargs.setdefault("arena", model.__dict__.get("_nestor_arena"))
        return MuonAdamW(build_param_groups(config, model), lr=config.lr_adamw, betas=config.betas,
                         eps=config.eps, weight_decay=config.weight_decay, momentum=config.muon_momentum,
                         nesterov=config.muon_nesterov, ns_steps=config.muon_ns_steps, **kwargs)
    params = [p for p in model.parameters() if p.requires_grad]
    if isinstance(config, AdamWConfig):
        return torch.optim.AdamW(params, lr=config.lr, betas=config.betas, eps=config.eps,
                                 weight_decay=config.weight_decay)
    if isinstance(config, AdamConfig):
        return torch.optim.Adam(params, lr=config.lr, betas=config.betas, eps=config.eps,
                                weight_decay=config.weight_decay)
    if isinstance(config, SGDConfig):
        return torch.optim.SGD(params, lr=config.lr, momentum=config.momentum, nesterov=config.nesterov,
                               weight_decay=config.weight_decay)
    raise TypeError(f"Unknown optimizer config {type(config).__name__}.")


def _with_warmup(opt: Optimizer, base: LRScheduler, warmup: int) -> LRScheduler:
    if warmup <= 0:
        return base
    ramp = LambdaLR(opt, lr_lambda=lambda step: step / max(1, warmup))
    return SequentialLR(opt, schedulers=[ramp, base], milestones=[warmup])


def build_scheduler(config: SchedulerConfig | None, opt: Optimizer,
                    num_training_steps: int | None = None) -> LRScheduler | None:
    """LR schedule factory (reference ``train/optim.py:340-490``).

    Cosine: linear warmup (``SequentialLR``) into ``CosineAnnealingLR(T_max, eta_min)`` where
    ``T_max`` counts from the end of warmup. WSD: warmup / stable / decay with the floor taken
    relative to the largest group lr. Power law: ``min(1, a/base_lr * (step*c)^b)`` with a
    linear ramp to that curve's value at the end of warmup.
    """

    if config is None:
        return None
    if isinstance(config, CosineAnnealingConfig):
        base = CosineAnnealingLR(opt, T_max=num_training_steps or config.T_max, eta_min=config.eta_min)
        return _with_warmup(opt, base, config.warmup_steps)
    if isinstance(config, StepLRConfig):
        return _with_warmup(opt, StepLR(opt, step_size=config.step_size, gamma=config.gamma), config.warmup_steps)
    if isinstance(config, WSDConfig):
        total = num_training_steps or config.total_steps
        warmup, decay = max(0, config.warmup_steps), max(1, config.decay_steps)
        decay_start = max(warmup, total - decay)
        lrs = [g["lr"] for g in opt.param_groups]
        top = max(lrs) if lrs else 1.0
        floor = config.eta_min / top if top > 0 else 0.0

        def wsd(step: int) -> float:
            if step < warmup:
                return step / max(1, warmup)
            if step < decay_start:
                return 1.0
            u = min(1.0, (step - decay_start) / decay)
            if config.decay_shape == "linear":
                tail = 1.0 - u
            elif config.decay_shape == "cosine":
                tail = 0.5 * (1.0 + math.cos(math.pi * u))
            else:
                tail = 1.0 - math.sqrt(u)
            return floor + (1.0 - floor) * tail

        return LambdaLR(opt, lr_lambda=wsd)
    if isinstance(config, PowerLawConfig):
        warmup = max(0, config.warmup_steps)

        def curve(step: int) -> float:
            return min(1.0, (config.a / config.base_lr) * ((max(1, step) * config.c) ** config.b))

        def power(step: int) -> float:
            if warmup > 0 and step <= warmup:
                return curve(warmup) * step / warmup
            return curve(step)

        return LambdaLR(opt, lr_lambda=power)
    raise TypeError(f"Unknown scheduler config {type(config).__name__}.")
