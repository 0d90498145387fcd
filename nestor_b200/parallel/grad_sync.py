"""Data-parallel gradient reduction over the parameter arena.

One reduction per optimizer step (gradients accumulate locally across micro-batches, as
the reference does with ``DDP.no_sync``, ``nestor/train/trainer.py:33-77``), averaging
over ranks. Two transports share the bucket walk:

* ``"fused"``: the peer-memory kernel of :mod:`nestor_b200.parallel.symm` — each rank
  reduces its slice of a bucket by loading the peers' slices over NVLink, scales by
  ``1/world``, writes fp32 (and optionally the bf16 cast) back to every replica.
* ``"nccl"`` / ``"gloo"``: ``torch.distributed.all_reduce`` on arena slices (the baseline,
  and the CPU test path).

Buckets are contiguous arena ranges, so no tensor is flattened or copied on either path.
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist

from nestor_b200.parallel.arena import ParamArena

DEFAULT_BUCKET_MB = 64


class GradReducer:
    def __init__(self, arena: ParamArena, *, transport: str | None = None, bucket_mb: int | None = None) -> None:
        self.arena = arena
        self.world = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
        self.rank = dist.get_rank() if self.world > 1 else 0
        mb = bucket_mb or int(os.environ.get("NESTOR_B200_BUCKET_MB", DEFAULT_BUCKET_MB))
        self.buckets = arena.buckets(mb * (1 << 20) // 4)
        if transport is None:
            transport = os.environ.get("NESTOR_B200_GRAD_TRANSPORT", "fused" if arena.grad.is_cuda else "gloo")
        self.transport = transport
        self._fused = None
        self._fused_rs = None
        if self.world > 1 and transport == "fused":
            from nestor_b200.parallel.symm import FusedAllReduce, FusedReduceScatter
            self._fused = FusedAllReduce(arena.grad, self.buckets)
            self._fused_rs = FusedReduceScatter(arena.grad, group=self._fused.group)

    @torch.no_grad()
    def reduce(self) -> None:
        """Average ``arena.grad`` over ranks in place."""

        if self.world == 1:
            return
        if self._fused is not None:
            self._fused.run(scale=1.0 / self.world)
            return
        works = []
        for off, n in self.buckets:
            works.append(dist.all_reduce(self.arena.grad[off : off + n], op=dist.ReduceOp.SUM, async_op=True))
        for w in works:
            w.wait()
        self.arena.grad.mul_(1.0 / self.world)

    @torch.no_grad()
    def reduce_scatter(self, lo: int, hi: int) -> None:
        """Average ``arena.grad[lo:hi]`` (this rank's ownership range) over ranks; the rest of the local
        gradient buffer keeps this rank's partial sums, which nothing reads (sharded optimizer)."""

        if self.world == 1:
            return
        if self._fused_rs is not None:
            self._fused_rs.run(lo, hi, 1.0 / self.world)
            return
        # library transports have no ragged reduce-scatter over arena ranges: reduce everything
        self.reduce()

    @torch.no_grad()
    def sync_buffers(self, model: torch.nn.Module, src: int = 0) -> None:
        """Broadcast every floating buffer (router ``choice_bias``) from ``src`` in one packed message."""

        if self.world == 1:
            return
        bufs = [b for _, b in model.named_buffers() if b.is_floating_point() and b.numel()]
        if not bufs:
            return
        flat = torch.cat([b.reshape(-1).float() for b in bufs])
        dist.broadcast(flat, src=src)
        off = 0
        for b in bufs:
            b.copy_(flat[off : off + b.numel()].view_as(b))
            off += b.numel()
