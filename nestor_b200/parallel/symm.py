"""Symmetric (peer-mapped) buffers and the fused collectives that run over them.

Buffers are allocated with ``torch.distributed._symmetric_memory`` (which exchanges the
CUDA memory handles over the process group) and the kernels of ``csrc/comm.cu`` then load
and store peer memory directly over NVLink: no NCCL call sits on the gradient-reduction or
parameter-distribution path. Flags for the in-kernel barriers live in a dedicated symmetric
``int32`` buffer (zero-initialised once; epochs only grow).

Every wait inside the kernels is bounded. ``check()`` reads the device status word and
raises ``PeerTimeout`` if a peer failed to arrive — the process group can then be torn
down by the caller instead of hanging.
"""

from __future__ import annotations

import ctypes as C
import os

import torch
import torch.distributed as dist

from nestor_b200.ops import _lib

MAX_WORLD = 8
PHASES = 4


def max_blocks() -> int:
    """Upper bound on the blocks of a collective launch: one per SM of this device."""

    return int(_L().nb_comm_max_blocks())


def nvls_wanted() -> bool:
    """``NESTOR_B200_NVLS``: ``auto`` (default) uses the NVLink multicast mapping whenever the symmetric buffers have
    one, ``0`` keeps every collective on plain peer loads and stores (failure-handling tests run that way: a rank must
    never die while its memory is bound to a multicast object)."""

    return os.environ.get("NESTOR_B200_NVLS", "auto") != "0"


class PeerTimeout(RuntimeError):
    """A bounded device-side wait on a peer flag gave up."""


class Peers(C.Structure):
    _fields_ = [("buf", C.c_void_p * 8), ("aux", C.c_void_p * 8), ("sig", C.c_void_p * 8),
                ("world", C.c_int), ("rank", C.c_int)]


_protos = False


def _L():
    global _protos
    L = _lib.lib()
    if not _protos:
        vp, i, l, f, u = C.c_void_p, C.c_int, C.c_long, C.c_float, C.c_uint
        L.nb_allreduce_push.argtypes = [C.POINTER(Peers), l, l, f, i, u, l, i, vp, vp]
        L.nb_reduce_scatter_push.argtypes = [C.POINTER(Peers), l, l, f, i, u, l, i, vp, vp]
        L.nb_reduce_scatter_push.restype = C.c_int
        L.nb_param_push.argtypes = [C.POINTER(Peers), l, l, u, l, i, vp, i, vp]
        L.nb_wait_timeout_probe.argtypes = [vp, u, l, vp, vp]
        L.nb_allreduce_nvls.argtypes = [C.POINTER(Peers), vp, vp, l, l, f, i, u, l, i, vp, vp]
        L.nb_reduce_scatter_nvls.argtypes = [C.POINTER(Peers), vp, l, l, f, i, u, l, i, vp, vp]
        L.nb_param_push_nvls.argtypes = [C.POINTER(Peers), vp, vp, l, l, u, l, i, vp, i, vp]
        L.nb_comm_max_blocks.argtypes = []
        for fn in (L.nb_allreduce_push, L.nb_param_push, L.nb_wait_timeout_probe, L.nb_allreduce_nvls,
                   L.nb_reduce_scatter_nvls, L.nb_param_push_nvls, L.nb_comm_max_blocks):
            fn.restype = C.c_int
        _protos = True
    return L


def symmetric_empty(numel: int, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
    """A flat tensor in symmetric memory (peer-mappable)."""

    import torch.distributed._symmetric_memory as symm_mem
    return symm_mem.empty(numel, dtype=dtype, device=device)


def rendezvous(t: torch.Tensor):
    import torch.distributed._symmetric_memory as symm_mem
    return symm_mem.rendezvous(t, dist.group.WORLD)


def wait_budget() -> int:
    """Polls (about 0.1-0.2 us each) a peer wait may spend; ``NESTOR_B200_PEER_WAIT_MS`` overrides (default 20 s)."""

    ms = float(os.environ.get("NESTOR_B200_PEER_WAIT_MS", "20000"))
    return max(1000, int(ms * 1e3 / 0.15))


class PeerGroup:
    """Peer pointers of up to two symmetric buffers plus the shared flag buffer."""

    _flags = None
    _flags_handle = None
    _epoch = 0

    def __init__(self, main: torch.Tensor, aux: torch.Tensor | None = None) -> None:
        self.world, self.rank = dist.get_world_size(), dist.get_rank()
        if self.world > MAX_WORLD:
            raise ValueError(f"fused collectives support up to {MAX_WORLD} ranks on one node")
        self.main, self.aux = main, aux
        self.h_main = rendezvous(main)
        self.h_aux = rendezvous(aux) if aux is not None else None
        if PeerGroup._flags is None:
            flags = symmetric_empty(PHASES * max_blocks() * MAX_WORLD, torch.int32, main.device)
            flags.zero_()
            torch.cuda.synchronize()
            PeerGroup._flags, PeerGroup._flags_handle = flags, rendezvous(flags)
            dist.barrier()
        self.peers = Peers()
        for r in range(self.world):
            self.peers.buf[r] = int(self.h_main.buffer_ptrs[r])
            self.peers.aux[r] = int(self.h_aux.buffer_ptrs[r]) if self.h_aux is not None else None
            self.peers.sig[r] = int(PeerGroup._flags_handle.buffer_ptrs[r])
        self.peers.world, self.peers.rank = self.world, self.rank
        self.blocks = min(int(os.environ.get("NESTOR_B200_COMM_BLOCKS", "64")), max_blocks())
        self.status = _lib.status_word(main.device)
        # NVLink multicast addresses of the two buffers (0 when the fabric or the allocation has none)
        self.mc_main = int(getattr(self.h_main, "multicast_ptr", 0) or 0) if nvls_wanted() else 0
        self.mc_aux = (int(getattr(self.h_aux, "multicast_ptr", 0) or 0) if self.h_aux is not None else 0) if nvls_wanted() else 0
        self.nvls = bool(self.mc_main) and (self.h_aux is None or bool(self.mc_aux))

    @classmethod
    def next_epoch(cls) -> int:
        cls._epoch = (cls._epoch + 1) & 0x7FFFFFFF
        return cls._epoch

    def check(self) -> None:
        code = int(self.status.item())
        if code:
            self.status.zero_()
            raise PeerTimeout(f"rank {self.rank}: a peer did not reach the in-kernel barrier (status {code})")


class FusedAllReduce:
    """Average a symmetric fp32 buffer over ranks in place, bucket by bucket, one kernel per bucket."""

    def __init__(self, grad: torch.Tensor, buckets: list[tuple[int, int]], mirror: torch.Tensor | None = None) -> None:
        self.group = PeerGroup(grad, mirror)
        self.buckets = buckets
        self.mirror = mirror is not None

    @torch.no_grad()
    def run(self, scale: float) -> None:
        g = self.group
        st = C.c_void_p(_lib.stream_ptr())
        budget = wait_budget()
        for off, n in self.buckets:
            n4 = (n // 4) * 4
            if g.nvls:
                rc = _L().nb_allreduce_nvls(C.byref(g.peers), g.mc_main, g.mc_aux or None, off, n4, scale, int(self.mirror),
                                            PeerGroup.next_epoch(), budget, g.blocks, g.status.data_ptr(), st)
            else:
                rc = _L().nb_allreduce_push(C.byref(g.peers), off, n4, scale, int(self.mirror), PeerGroup.next_epoch(), budget,
                                            g.blocks, g.status.data_ptr(), st)
            if rc != 0:
                raise RuntimeError(f"fused all-reduce launch failed with code {rc}")
            _lib.count_launch()
            if n4 != n:   # ragged tail (arena sizes are multiples of 64, so this is for ad-hoc buffers only)
                tail = g.main[off + n4 : off + n]
                dist.all_reduce(tail)
                tail.mul_(scale)


class FusedReduceScatter:
    """Sum a symmetric fp32 buffer over ranks, each rank keeping only the range it owns (one kernel)."""

    def __init__(self, grad: torch.Tensor, mirror: torch.Tensor | None = None, group: PeerGroup | None = None) -> None:
        self.group = group if group is not None else PeerGroup(grad, mirror)   # may share the all-reduce's peer table
        self.mirror = self.group.aux is not None

    @torch.no_grad()
    def run(self, lo: int, hi: int, scale: float) -> None:
        g = self.group
        assert lo % 4 == 0 and hi % 4 == 0
        if g.nvls:
            rc = _L().nb_reduce_scatter_nvls(C.byref(g.peers), g.mc_main, lo, hi, scale, int(self.mirror), PeerGroup.next_epoch(),
                                             wait_budget(), g.blocks, g.status.data_ptr(), C.c_void_p(_lib.stream_ptr()))
        else:
            rc = _L().nb_reduce_scatter_push(C.byref(g.peers), lo, hi, scale, int(self.mirror), PeerGroup.next_epoch(),
                                             wait_budget(), g.blocks, g.status.data_ptr(), C.c_void_p(_lib.stream_ptr()))
        if rc != 0:
            raise RuntimeError(f"fused reduce-scatter launch failed with code {rc}")
        _lib.count_launch()


class ParamPush:
    """After a sharded optimizer step: store the bf16 cast of this rank's master range into every replica's compute
    copy, and (``push_master``) the fp32 values into every replica's master too.

    ``push_master=None`` reads ``NESTOR_B200_PUSH_MASTER`` (default 0): only the compute copy travels, 2 bytes per
    parameter instead of 6; fp32 masters outside a rank's own range then go stale until ``gather_masters`` brings them
    up to date from their owners (checkpoints, comparisons). Without a separate compute copy (fp32 compute) the master
    is what is pushed.
    """

    def __init__(self, master: torch.Tensor, compute: torch.Tensor | None, push_master: bool | None = None) -> None:
        self.group = PeerGroup(master, compute if compute is not None and compute is not master else None)
        if push_master is None:
            push_master = os.environ.get("NESTOR_B200_PUSH_MASTER", "0") == "1"
        self.push_master = bool(push_master) or self.group.aux is None
        # A multicast store also lands in the sender's own copy, so on few ranks it moves more bytes than the
        # world - 1 peer stores it replaces (measured on 2 GPUs: 330 vs 609 GB/s); it pays from 4 ranks on.
        self.use_nvls = self.group.nvls and self.group.world >= int(os.environ.get("NESTOR_B200_NVLS_PUSH_MIN_WORLD", "4"))

    @torch.no_grad()
    def run(self, lo: int, hi: int) -> None:
        g = self.group
        if self.use_nvls:
            rc = _L().nb_param_push_nvls(C.byref(g.peers), g.mc_main, g.mc_aux or None, lo, hi, PeerGroup.next_epoch(),
                                         wait_budget(), g.blocks, g.status.data_ptr(), int(self.push_master),
                                         C.c_void_p(_lib.stream_ptr()))
        else:
            rc = _L().nb_param_push(C.byref(g.peers), lo, hi, PeerGroup.next_epoch(), wait_budget(), g.blocks,
                                    g.status.data_ptr(), int(self.push_master), C.c_void_p(_lib.stream_ptr()))
        if rc != 0:
            raise RuntimeError(f"fused parameter push launch failed with code {rc}")
        _lib.count_launch()


@torch.no_grad()
def gather_ranges(flat: torch.Tensor, cuts: list[int]) -> None:
    """Bring ``flat`` up to date on every rank from the owners of its ranges: rank ``r`` broadcasts
    ``flat[cuts[r]:cuts[r + 1]]`` (control-plane collective; used when a checkpoint or a comparison needs the whole
    fp32 state that the training step keeps sharded)."""

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return
    for r in range(dist.get_world_size()):
        lo, hi = cuts[r], cuts[r + 1]
        if hi > lo:
            dist.broadcast(flat[lo:hi], src=r)


def wait_timeout_probe(device: torch.device, budget: int = 20000) -> int:
    """Run the single-GPU bounded-wait probe (a flag nothing sets); returns the status code the kernel left."""

    flag = torch.zeros(1, dtype=torch.int32, device=device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    rc = _L().nb_wait_timeout_probe(flag.data_ptr(), 1, budget, status.data_ptr(), C.c_void_p(_lib.stream_ptr()))
    if rc != 0:
        raise RuntimeError(f"nb_wait_timeout_probe failed with code {rc}")
    torch.cuda.synchronize(device)
    return int(status.item())
