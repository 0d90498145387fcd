"""ctypes binding of the in-tree sm_100a kernel library.

The library lives at ``nestor_b200/_C/libnestor_b200.so`` and is brought up to date on first use
(objects are cached by source digest, so nothing is recompiled when nothing changed). Without a
compiler a stale or missing library is an error: there is no silent PyTorch fallback for CUDA
tensors, and a binary older than the ctypes structures of this package is never loaded.
"""

from __future__ import annotations

import ctypes as C
from pathlib import Path

import torch

_LIB = None
LAUNCHES = 0   # kernels of this library launched so far (bench.py reports the delta)


class Operand(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("rows", C.c_long), ("cols", C.c_long), ("ld", C.c_long),
                ("groups", C.c_long), ("group_stride", C.c_long)]


class GemmArgs(C.Structure):
    _fields_ = [
        ("mode", C.c_int), ("groups", C.c_int), ("BN", C.c_int), ("epilogue", C.c_int),
        ("M", C.c_int), ("N", C.c_int), ("K", C.c_int), ("K2", C.c_int),
        ("offsets", C.c_void_p), ("rows_per_group", C.c_int),
        ("a_mn", C.c_int), ("b_mn", C.c_int), ("b_grouped", C.c_int),
        ("A", Operand), ("B", Operand), ("A2", Operand), ("B2", Operand),
        ("C", C.c_void_p), ("ldc", C.c_long), ("c_group_stride", C.c_long),
        ("C2", C.c_void_p), ("C3", C.c_void_p), ("E1", C.c_void_p), ("E2", C.c_void_p), ("lde", C.c_long),
        ("alpha", C.c_float), ("beta", C.c_float), ("n_valid", C.c_int), ("splits", C.c_int), ("status", C.c_void_p),
        ("max_m_tiles", C.c_int),
        ("sms", C.c_int), ("trace", C.c_void_p),
        ("prefetch_dist", C.c_int), ("prefetch_ops", C.c_int), ("max_stages", C.c_int), ("pair", C.c_int), ("debug", C.c_int),
        # fused all-gather of B / B2 (csrc/gemm.cu: GatherParams)
        ("gather_src", C.c_void_p * 8), ("gather_dst", C.c_void_p),
        ("gather_seg_src_off", C.c_long * 2), ("gather_seg_dst_off", C.c_long * 2),
        ("gather_group_bytes", C.c_long), ("gather_group_stride_src", C.c_long),
        ("gather_nseg", C.c_int), ("gather_groups_per_rank", C.c_int), ("gather_on", C.c_int), ("gather_chunk", C.c_int),
        ("gather_flags", C.c_void_p), ("gather_nbuf", C.c_int), ("gather_lanes", C.c_int),
        ("gather_wait_polls", C.c_uint),
        ("no_tiled_store", C.c_int),
    ]


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        # always go through the build front end: unchanged sources cost a hash, changed ones are recompiled, and a
        # machine without a compiler refuses a binary that is older than its sources
        # NESTOR_B200_BOUNDS_CHECK=1 loads the index-checking build of the same sources (gather-style kernels record an
        # out-of-range index in a status record instead of reading through it; ops.cuda.bounds_check_report())
        import os
        from nestor_b200.csrc.build import ensure
        _LIB = C.CDLL(str(ensure(checked=os.environ.get("NESTOR_B200_BOUNDS_CHECK") == "1")))
        _LIB.nb_gemm.argtypes = [C.POINTER(GemmArgs), C.c_void_p]
        _LIB.nb_gemm.restype = C.c_int
    return _LIB


_sms: dict[int, int] = {}


def sm_count(device: torch.device | None = None) -> int:
    """Streaming multiprocessors of ``device`` (grids and split factors are sized from it)."""

    idx = torch.cuda.current_device() if device is None or device.index is None else device.index
    if idx not in _sms:
        _sms[idx] = int(torch.cuda.get_device_properties(idx).multi_processor_count)
    return _sms[idx]


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def count_launch(n: int = 1) -> None:
    global LAUNCHES
    LAUNCHES += n


_status: dict[int, torch.Tensor] = {}


def status_word(device: torch.device) -> torch.Tensor:
    """Per-device int32 the kernels write a nonzero code into when a bounded wait gives up."""

    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _status:
        _status[idx] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status[idx]


def check_status(device: torch.device) -> None:
    """Raise if any kernel on ``device`` reported a timed-out wait (synchronises)."""

    code = int(status_word(device).item())
    if code:
        status_word(device).zero_()
        raise RuntimeError(f"nestor_b200 kernel reported status {code} (a bounded device-side wait gave up)")


class FlashArgs(C.Structure):
    _fields_ = [
        ("Q", C.c_void_p), ("K", C.c_void_p), ("V", C.c_void_p), ("ld_qkv", C.c_long),
        ("O", C.c_void_p), ("ldo", C.c_long), ("lse", C.c_void_p),
        ("seg_start", C.c_void_p), ("nseg", C.c_int),
        ("rows", C.c_int), ("H", C.c_int), ("hd", C.c_int), ("scale", C.c_float),
        ("status", C.c_void_p), ("max_tiles", C.c_int), ("lazy_rescale", C.c_int),
    ]


class FlashBwdArgs(C.Structure):
    _fields_ = [
        ("Q", C.c_void_p), ("K", C.c_void_p), ("V", C.c_void_p), ("ld_qkv", C.c_long),
        ("O", C.c_void_p), ("ld_o", C.c_long), ("dO", C.c_void_p), ("ld_do", C.c_long),
        ("lse", C.c_void_p), ("delta", C.c_void_p),
        ("dQ", C.c_void_p), ("dK", C.c_void_p), ("dV", C.c_void_p), ("ld_dqkv", C.c_long),
        ("seg_start", C.c_void_p), ("nseg", C.c_int),
        ("rows", C.c_int), ("H", C.c_int), ("hd", C.c_int), ("scale", C.c_float),
        ("status", C.c_void_p), ("max_tiles", C.c_int),
    ]
