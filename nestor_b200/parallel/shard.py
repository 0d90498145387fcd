"""Rank-sharded expert banks read through the all-gather fused into the grouped GEMM.

With ``NESTOR_FSDP_BANKS=1`` the expert-bank products of a data-parallel run stop reading the local bf16
copy of the banks: rank ``r`` is the owner of experts ``[r * E / W, (r + 1) * E / W)`` of every bank, and each
product that consumes a bank stages the experts from their owners' weight arenas (which every rank maps through
symmetric memory) inside the GEMM launch itself — a copy warp in every CTA pulls the shards over NVLink with bulk
copies while the other warps already multiply the experts that have arrived (``csrc/gemm.cu``: ``GatherParams``). The
staging buffer holds one product's banks only and is reused by the next product, forward and backward alike
(the "reshard after forward" policy of the reference's FSDP2 wrapping, ``nestor/utils/distributed.py:445-489``).

The fp32 master copy, its gradient and the replicated bf16 arena are still allocated per rank in this mode
(the optimizer state is what is sharded, see ``train/optim.py``); what the mode provides is the fused
all-gather -> GEMM data path and its measurement, the piece a parameter-sharded arena would be built on.
"""

from __future__ import annotations

import os

import torch
from torch import Tensor

from nestor_b200.ops import gemm as G

MAX_GROUPS = 256


class ShardedBanks:
    """Hands ``ops.gemm.Gather`` descriptions to the expert-bank products of one device."""

    def __init__(self, compute: Tensor, peer_ptrs: list[int], rank: int) -> None:
        self.compute, self.peer_ptrs, self.rank, self.world = compute, list(peer_ptrs), rank, len(peer_ptrs)
        self.lo = compute.data_ptr()
        self.hi = self.lo + compute.numel() * compute.element_size()
        self.chunk = int(os.environ.get("NESTOR_FSDP_GATHER_CHUNK", "8192"))
        self.nbuf = int(os.environ.get("NESTOR_FSDP_GATHER_NBUF", "4"))
        self.flags = torch.zeros(MAX_GROUPS + 1, dtype=torch.int32, device=compute.device)
        self.stage: Tensor | None = None
        self.gathered_bytes = 0       # bytes staged since construction (host-side count, for reports)

    def _fits(self, w: Tensor) -> bool:
        return (w.ndim == 3 and w.dtype == torch.bfloat16 and w.shape[0] % self.world == 0 and w.shape[0] <= MAX_GROUPS
                and w[0].is_contiguous() and self.lo <= w.data_ptr() < self.hi
                and (w.shape[1] * w.shape[2] * 2) % 16 == 0 and (w.stride(0) * 2) % 16 == 0
                and (w.data_ptr() - self.lo) % 16 == 0)

    def spec(self, w: Tensor, w2: Tensor | None = None) -> G.Gather | None:
        """Gather description for a product whose B operand is ``w`` (and ``w2``), or ``None`` to read locally."""

        if self.world < 2 or not self._fits(w) or (w2 is not None and not (self._fits(w2) and w2.shape == w.shape
                                                                           and w2.stride() == w.stride())):
            return None
        need = w.numel() * 2 * (2 if w2 is not None else 1)
        if self.stage is None or self.stage.numel() * 2 < need:
            self.stage = torch.empty(need // 2, dtype=torch.bfloat16, device=w.device)
        self.gathered_bytes += need
        return G.Gather(src=self.peer_ptrs, arena_ptr=self.lo, stage=self.stage, flags=self.flags,
                        groups_per_rank=w.shape[0] // self.world, chunk=self.chunk, nbuf=self.nbuf)
