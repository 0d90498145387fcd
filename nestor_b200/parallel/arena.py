"""Flat parameter arena: one fp32 master buffer, one fp32 gradient buffer, one compute copy.

The trainable parameters of a model are re-homed as views into three flat buffers of
identical layout:

* ``master`` (fp32): what the optimizer updates and what checkpoints store.
* ``grad`` (fp32): every ``p.grad`` is a view here, so zeroing gradients is one memset,
  the gradient norm is one reduction, and the data-parallel reduction walks the buffer in
  fixed-size buckets with no flatten/unflatten copies.
* ``compute`` (bf16 on GPUs; an alias of ``master`` when the compute dtype is fp32): what
  GEMM kernels read. It is refreshed once per optimizer step (not per micro-batch) by one
  cast over the whole buffer, or written directly by the fused parameter-distribution
  kernel after a sharded optimizer step.

Parameters keep their ``state_dict`` names and shapes. They are laid out in
``named_parameters()`` order with each tensor's offset aligned to ``ALIGN`` elements, so
the per-column attention projections of a layer sit at a constant stride and can be
viewed as one ``[G, rows, cols]`` operand (``stack_view``) without copying.

The reference keeps ordinary per-tensor parameters under DDP's bucket views
(``nestor/utils/distributed.py:436-443``, ``gradient_as_bucket_view=True``) and casts
weights under autocast on every use; this arena replaces both mechanisms.
"""

from __future__ import annotations

import dataclasses as dc
from typing import Iterable

import torch
from torch import Tensor, nn

ALIGN = 64  # elements: 256 B of fp32, 128 B of bf16 — keeps every view 16-byte aligned for TMA


@dc.dataclass
class Slot:
    name: str
    offset: int
    numel: int
    shape: torch.Size


class _ComputeView(torch.autograd.Function):
    """Hand a compute-dtype view to the graph; route its gradient to the fp32 parameters."""

    @staticmethod
    def forward(ctx, view: Tensor, *params: Tensor) -> Tensor:
        ctx.shapes = [p.shape for p in params]
        ctx.dtypes = [p.dtype for p in params]
        # kernels that add a weight gradient straight into the arena return no gradient for the view: without this
        # autograd would materialise a zero tensor and add it to every parameter behind the view
        ctx.set_materialize_grads(False)
        return view.detach()

    @staticmethod
    def backward(ctx, grad: Tensor):
        if grad is None:
            return (None,) * (1 + len(ctx.shapes))
        if len(ctx.shapes) == 1:
            return None, grad.reshape(ctx.shapes[0]).to(ctx.dtypes[0])
        if grad.shape[0] == len(ctx.shapes):          # stack of same-shape parameters
            return (None, *[g.reshape(s).to(dt) for g, s, dt in zip(grad.unbind(0), ctx.shapes, ctx.dtypes)])
        per = len(ctx.shapes) // grad.shape[0]        # fused groups: split each group's rows
        outs = []
        for gi, g in enumerate(grad.unbind(0)):
            r = 0
            for s, dt in zip(ctx.shapes[gi * per : (gi + 1) * per], ctx.dtypes[gi * per : (gi + 1) * per]):
                outs.append(g[r : r + s[0]].reshape(s).to(dt))
                r += s[0]
        return (None, *outs)


class ParamArena:
    def __init__(self, model: nn.Module, *, compute_dtype: torch.dtype = torch.float32,
                 device: torch.device | None = None, symmetric: bool = False) -> None:
        named = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
        if not named:
            raise ValueError("model has no trainable parameters")
        device = device or named[0][1].device
        self.compute_dtype = compute_dtype
        self.slots: dict[str, Slot] = {}
        self._slot_of: dict[int, Slot] = {}
        off = 0
        for n, p in named:
            s = Slot(n, off, p.numel(), p.shape)
            self.slots[n] = s
            self._slot_of[id(p)] = s
            off += -(-p.numel() // ALIGN) * ALIGN
        self.numel = off
        self.symmetric = symmetric

        def alloc(dtype: torch.dtype) -> Tensor:
            if symmetric:   # peer-mappable memory for the in-kernel collectives
                from nestor_b200.parallel.symm import symmetric_empty
                return symmetric_empty(off, dtype, device).zero_()
            return torch.zeros(off, dtype=dtype, device=device)

        self.master = alloc(torch.float32)
        self.grad = alloc(torch.float32)
        with torch.no_grad():
            for n, p in named:
                s = self.slots[n]
                view = self.master[s.offset : s.offset + s.numel].view(s.shape)
                view.copy_(p.detach().to(device=device, dtype=torch.float32))
                p.data = view
                p.grad = self.grad[s.offset : s.offset + s.numel].view(s.shape)
        self.compute = self.master if compute_dtype == torch.float32 else alloc(compute_dtype)
        self.params = [p for _, p in named]
        self.refresh_compute()
        for m in model.modules():  # discoverable from every module that owns parameters
            m.__dict__["_nestor_arena"] = self

    # ------------------------------------------------------------------------ views
    def slot(self, p: Tensor) -> Slot:
        return self._slot_of[id(p)]

    @torch.no_grad()
    def refresh_compute(self) -> None:
        """Re-derive the compute copy from the masters (one cast over the flat buffer)."""

        if self.compute is not self.master:
            self.compute.copy_(self.master)

    def zero_grad(self) -> None:
        self.grad.zero_()

    def compute_view(self, p: Tensor) -> Tensor:
        """Compute-dtype weight of ``p`` wired into autograd (gradient lands in ``p.grad``).

        The returned tensor carries ``_nb_grad``: the fp32 gradient view a kernel may accumulate
        into directly (returning no gradient through autograd for that operand).
        """

        if self.compute is self.master:
            return p
        s = self.slot(p)
        return self._wire(self.compute[s.offset : s.offset + s.numel].view(s.shape),
                          self.grad[s.offset : s.offset + s.numel].view(s.shape), [p])

    def _wire(self, view: Tensor, grad_view: Tensor, params: list[Tensor]) -> Tensor:
        out = _ComputeView.apply(view, *params) if torch.is_grad_enabled() and params[0].requires_grad else view
        out._nb_grad = grad_view
        return out

    def _strided(self, slots: list[Slot]) -> tuple[int, bool]:
        stride = slots[1].offset - slots[0].offset if len(slots) > 1 else slots[0].numel
        ok = all(b.offset - a.offset == stride for a, b in zip(slots[:-1], slots[1:]))
        return stride, ok

    def stack_view(self, params: Iterable[Tensor]) -> Tensor:
        """``[n, *shape]`` operand over ``n`` same-shape parameters at a constant stride (no copy)."""

        params = list(params)
        slots = [self.slot(p) for p in params]
        shape = slots[0].shape
        stride, ok = self._strided(slots)
        ok = ok and all(s.shape == shape for s in slots)
        if not ok or self.compute is self.master:
            return torch.stack([self.compute_view(p) for p in params], dim=0)
        inner = list(torch.empty(shape, device="meta").stride())
        geom = ((len(params), *shape), (stride, *inner), slots[0].offset)
        return self._wire(torch.as_strided(self.compute, *geom), torch.as_strided(self.grad, *geom), params)

    def fused_view(self, groups: list[list[Tensor]]) -> Tensor:
        """``[G, sum(rows), cols]`` operand where group ``g`` is the row-concatenation of ``groups[g]``.

        Requires the members of a group to be adjacent in the arena (each ``[rows_i, cols]`` with
        ``rows_i * cols`` a multiple of the arena alignment) and the groups to sit at a constant
        stride — true for the per-column ``q_proj, k_proj, v_proj`` triples. Falls back to a copy.
        """

        flat = [p for g in groups for p in g]
        cols = flat[0].shape[-1]
        rows = sum(p.shape[0] for p in groups[0])
        firsts = [self.slot(g[0]) for g in groups]
        stride, ok = self._strided(firsts)
        for g in groups:
            off = self.slot(g[0]).offset
            for p in g:
                ok = ok and self.slot(p).offset == off and p.shape[-1] == cols
                off += p.numel()
        if not ok or self.compute is self.master:
            return torch.stack([torch.cat([self.compute_view(p) for p in g], dim=0) for g in groups], dim=0)
        geom = ((len(groups), rows, cols), (stride, cols, 1), firsts[0].offset)
        out = self._wire(torch.as_strided(self.compute, *geom), torch.as_strided(self.grad, *geom), flat)
        return out

    def concat_view(self, params: Iterable[Tensor]) -> Tensor:
        """``[sum(rows), cols]`` operand over row-adjacent 2-D parameters (one GEMM for several heads)."""

        params = list(params)
        v = self.fused_view([params])
        out = v[0]
        g = getattr(v, "_nb_grad", None)
        if g is not None:
            out._nb_grad = g[0]
        return out

    def buckets(self, bucket_elems: int) -> list[tuple[int, int]]:
        """``[(offset, numel)]`` covering the arena in order, each at most ``bucket_elems`` long."""

        out, off = [], 0
        while off < self.numel:
            n = min(bucket_elems, self.numel - off)
            out.append((off, n))
            off += n
        return out


def arena_of(module: nn.Module) -> ParamArena | None:
    return module.__dict__.get("_nestor_arena")
