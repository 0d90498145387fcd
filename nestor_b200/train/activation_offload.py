"""Spill saved activations to pinned host memory while a step is over its device budget.

``with activation_offload():`` installs ``saved_tensors_hooks`` around a forward pass. A saved
CUDA tensor is moved to pinned host memory on a copy stream when (a) it is at least
``NESTOR_ACTIVATION_OFFLOAD_MIN_MIB`` (default 1 MiB), (b) the device currently holds more than
``NESTOR_ACTIVATION_OFFLOAD_GIB`` (default 80 % of the device), and (c) the host budget
``NESTOR_ACTIVATION_OFFLOAD_MAX_GIB`` (default 16) is not exhausted. Views of one storage share
a single host copy (keyed by storage pointer, size, dtype and version) as long as the storage is
at most 16x the view, so the many reads of the same depth sources are spilled once. The
backward pass brings tensors back on demand. Parameters and non-CUDA tensors are never moved.
Enable from the trainer with ``NESTOR_ACTIVATION_OFFLOAD=1``. Behavioural parity with
``nestor/train/activation_offload.py:277-381`` (context), ``:128-199`` (storage-keyed cache).
"""

from __future__ import annotations

import os
import weakref
from contextlib import contextmanager
from typing import Any, Iterator

import torch
from torch import Tensor

GIB, MIB = 2**30, 2**20
SHARE_STORAGE_RATIO = 16


class ActivationOffloadStats:
    def __init__(self) -> None:
        self.packed = self.passed = self.bytes_moved = self.shared = 0

    def summary(self) -> str:
        if not self.packed:
            return f"offload: nothing moved ({self.passed} tensors stayed resident)"
        return (f"offload: {self.packed} tensors / {self.bytes_moved / GIB:.2f} GiB to host "
                f"({self.passed} stayed resident, {self.shared} saves shared a copy)")


class _HostCopy:
    """One pinned host copy of a whole device storage."""

    __slots__ = ("host", "device", "ready", "__weakref__")

    def __init__(self, host: Tensor, device: torch.device, ready: torch.cuda.Event) -> None:
        self.host, self.device, self.ready = host, device, ready


class _View:
    """How to rebuild one saved tensor from a host copy of its storage."""

    __slots__ = ("copy", "offset", "shape", "stride", "dtype")

    def __init__(self, copy: _HostCopy, t: Tensor) -> None:
        self.copy, self.offset, self.shape, self.stride, self.dtype = copy, t.storage_offset(), t.shape, t.stride(), t.dtype


class HostCopyCache:
    """Host copies keyed by storage identity; entries die with their last referencing save."""

    def __init__(self) -> None:
        self._by_key: "weakref.WeakValueDictionary[tuple, _HostCopy]" = weakref.WeakValueDictionary()

    @staticmethod
    def key(t: Tensor) -> tuple:
        s = t.untyped_storage()
        return (s.data_ptr(), s.nbytes(), t.dtype, t._version)

    def get(self, t: Tensor) -> _HostCopy | None:
        return self._by_key.get(self.key(t))

    def put(self, t: Tensor, copy: _HostCopy) -> None:
        self._by_key[self.key(t)] = copy


def _env_gib(name: str, default: float) -> float:
    v = os.environ.get(name)
    return float(v) if v else default


@contextmanager
def activation_offload(stats: ActivationOffloadStats | None = None) -> Iterator[ActivationOffloadStats]:
    stats = stats or ActivationOffloadStats()
    if not torch.cuda.is_available():
        yield stats
        return
    dev = torch.cuda.current_device()
    total = torch.cuda.get_device_properties(dev).total_memory
    trigger = _env_gib("NESTOR_ACTIVATION_OFFLOAD_GIB", 0.8 * total / GIB) * GIB
    floor = _env_gib("NESTOR_ACTIVATION_OFFLOAD_MIN_MIB", 1.0) * MIB
    host_cap = _env_gib("NESTOR_ACTIVATION_OFFLOAD_MAX_GIB", 16.0) * GIB
    cache = HostCopyCache()
    copy_stream = torch.cuda.Stream()
    host_bytes = 0

    def pack(t: Tensor) -> Any:
        nonlocal host_bytes
        if (not t.is_cuda or isinstance(t, torch.nn.Parameter) or t.numel() * t.element_size() < floor
                or torch.cuda.memory_allocated(dev) < trigger):
            stats.passed += 1
            return t
        hit = cache.get(t)
        if hit is not None:
            stats.shared += 1
            return _View(hit, t)
        storage_bytes = t.untyped_storage().nbytes()
        view_bytes = t.numel() * t.element_size()
        whole = storage_bytes <= SHARE_STORAGE_RATIO * view_bytes
        src = torch.empty(0, dtype=t.dtype, device=t.device).set_(t.untyped_storage()) if whole else t.contiguous()
        nbytes = src.numel() * src.element_size()
        if host_bytes + nbytes > host_cap:
            stats.passed += 1
            return t
        host = torch.empty(src.shape, dtype=src.dtype, pin_memory=True)
        copy_stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(copy_stream):
            host.copy_(src, non_blocking=True)
            ready = torch.cuda.Event()
            ready.record(copy_stream)
        src.record_stream(copy_stream)
        copy = _HostCopy(host, t.device, ready)
        host_bytes += nbytes
        stats.packed += 1
        stats.bytes_moved += nbytes
        if whole:
            cache.put(t, copy)
            return _View(copy, t)
        v = _View(copy, src)
        v.offset, v.shape, v.stride = 0, t.shape, src.stride()
        return v

    def unpack(obj: Any) -> Tensor:
        if not isinstance(obj, _View):
            return obj
        obj.copy.ready.synchronize()
        flat = obj.copy.host.to(obj.copy.device, non_blocking=True)
        return torch.as_strided(flat.view(-1) if flat.ndim != 1 else flat, obj.shape, obj.stride, obj.offset)

    with torch.autograd.graph.saved_tensors_hooks(pack, unpack):
        yield stats
