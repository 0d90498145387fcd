"""Multi-tensor optimizer launches (``csrc/optim.cu``): one kernel per parameter group and operation.

A group's tensor table (base pointers + element counts) and chunk list live on the device and are cached for as
long as the group's tensors keep their addresses (arena views and optimizer state never move).
"""

from __future__ import annotations

import ctypes as C

import torch
from torch import Tensor

from nestor_b200.ops import _lib

ADAMW, MOMENTUM, AXPY_F32, AXPY_BF16 = range(4)
_cache: dict[tuple, tuple[Tensor, Tensor, int]] = {}
_proto = False


def available(t: Tensor) -> bool:
    return t.is_cuda


def _tables(lists: list[list[Tensor]]) -> tuple[Tensor, Tensor, int]:
    key = tuple(t.data_ptr() for ts in lists for t in ts) + (len(lists),)
    hit = _cache.get(key)
    if hit is not None:
        return hit
    L = _lib.lib()
    chunk = L.nb_multi_tensor_chunk()
    n = len(lists[0])
    rows, chunks = [], []
    for i in range(n):
        numel = lists[0][i].numel()
        ptrs = [ts[i].data_ptr() for ts in lists] + [0] * (4 - len(lists))
        rows.append(ptrs + [numel])
        chunks.extend([i, c] for c in range(-(-numel // chunk)))
    dev = lists[0][0].device
    table = torch.tensor(rows, dtype=torch.int64).to(dev)
    ch = torch.tensor(chunks, dtype=torch.int32).to(dev) if chunks else torch.zeros(0, 2, dtype=torch.int32, device=dev)
    out = (table, ch, len(chunks))
    if len(_cache) > 256:
        _cache.clear()
    _cache[key] = out
    return out


def launch(op: int, lists: list[list[Tensor]], scalars: list[float]) -> None:
    """``lists``: up to four equally long tensor lists (all contiguous, fp32 unless the op says otherwise)."""

    global _proto
    if not lists or not lists[0]:
        return
    for ts in lists:
        for t in ts:
            assert t.is_contiguous(), "multi-tensor kernels index tensors linearly"
    table, chunks, n_chunks = _tables(lists)
    L = _lib.lib()
    if not _proto:
        L.nb_multi_tensor.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.POINTER(C.c_float), C.c_void_p]
        L.nb_multi_tensor.restype = C.c_int
        _proto = True
    sc = (C.c_float * 8)(*(list(scalars) + [0.0] * (8 - len(scalars))))
    rc = L.nb_multi_tensor(op, table.data_ptr(), chunks.data_ptr(), n_chunks, sc, C.c_void_p(_lib.stream_ptr()))
    if rc != 0:
        raise RuntimeError(f"nb_multi_tensor failed with code {rc}")
    _lib.count_launch()
