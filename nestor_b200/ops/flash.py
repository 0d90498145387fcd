"""Python front end of the varlen causal flash-attention kernels (``csrc/flash_*.cu``)."""

from __future__ import annotations

import ctypes as C
import os

import torch
from torch import Tensor

from nestor_b200.ops import _lib

# Forward variant: keep the output accumulator in TMEM across kv tiles and rescale it only when a row maximum moves by
# more than 2^8 (1), or fold it into registers after every tile (0).
LAZY_RESCALE = os.environ.get("NESTOR_B200_FLASH_LAZY", "1") == "1"
# head dims <= 64: the softmax warps hand the probabilities to the P V product through tensor memory (tcgen05.st, A
# operand of the MMA read from TMEM) instead of a swizzled shared-memory tile; "0" keeps the shared-memory path
P_IN_TMEM = os.environ.get("NESTOR_B200_FLASH_P_TMEM", "1") == "1"


def flash_fwd(q: Tensor, k: Tensor, v: Tensor, seg_start: Tensor, heads: int, head_dim: int, scale: float,
              out: Tensor | None = None) -> tuple[Tensor, Tensor]:
    """Causal attention inside each packed segment.

    ``q, k, v``: bf16 ``[rows, >= heads*head_dim]`` views with one shared row pitch (e.g. the three
    column ranges of a fused qkv buffer); head ``h`` occupies columns ``h*head_dim ..``. Returns
    ``(out [rows, heads*head_dim] bf16, lse [rows, heads] fp32 in the log2 domain)``.
    """

    rows = q.shape[0]
    ld = q.stride(0)
    assert k.stride(0) == ld and v.stride(0) == ld and q.stride(1) == 1
    assert q.dtype == torch.bfloat16 and head_dim % 8 == 0
    for t in (q, k, v):
        assert t.data_ptr() % 16 == 0 and (ld * 2) % 16 == 0
    if out is None:
        out = torch.empty(rows, heads * head_dim, dtype=torch.bfloat16, device=q.device)
    lse = torch.empty(rows, heads, dtype=torch.float32, device=q.device)
    nseg = seg_start.numel() - 1
    a = _lib.FlashArgs()
    a.Q, a.K, a.V, a.ld_qkv = q.data_ptr(), k.data_ptr(), v.data_ptr(), ld
    a.O, a.ldo, a.lse = out.data_ptr(), out.stride(0), lse.data_ptr()
    a.seg_start, a.nseg = seg_start.data_ptr(), nseg
    a.rows, a.H, a.hd, a.scale = rows, heads, head_dim, scale
    a.status = _lib.status_word(q.device).data_ptr()
    a.max_tiles = -(-rows // 128) + nseg
    a.lazy_rescale = int(LAZY_RESCALE) | (2 if P_IN_TMEM else 0)
    L = _lib.lib()
    L.nb_flash_fwd.argtypes = [C.POINTER(_lib.FlashArgs), C.c_void_p]
    L.nb_flash_fwd.restype = C.c_int
    rc = L.nb_flash_fwd(C.byref(a), C.c_void_p(_lib.stream_ptr()))
    if rc != 0:
        raise RuntimeError(f"nb_flash_fwd failed with code {rc}")
    _lib.count_launch()
    return out, lse


def flash_bwd(q: Tensor, k: Tensor, v: Tensor, o: Tensor, do: Tensor, lse: Tensor, seg_start: Tensor,
              heads: int, head_dim: int, scale: float, dqkv: Tensor | None = None) -> Tensor:
    """Gradients of :func:`flash_fwd`. Returns one ``[rows, 3*heads*head_dim]`` bf16 buffer ``[dQ | dK | dV]``.

    Launches three kernels: the ``delta = rowsum(dO * O)`` reduction, the dK/dV pass and the dQ pass.
    """

    rows = q.shape[0]
    inner = heads * head_dim
    ld = q.stride(0)
    assert k.stride(0) == ld and v.stride(0) == ld
    assert do.dtype == torch.bfloat16 and do.stride(1) == 1 and (do.stride(0) * 2) % 16 == 0 and do.data_ptr() % 16 == 0
    if dqkv is None:
        dqkv = torch.empty(rows, 3 * inner, dtype=torch.bfloat16, device=q.device)
    delta = torch.empty(rows, heads, dtype=torch.float32, device=q.device)
    nseg = seg_start.numel() - 1
    a = _lib.FlashBwdArgs()
    a.Q, a.K, a.V, a.ld_qkv = q.data_ptr(), k.data_ptr(), v.data_ptr(), ld
    a.O, a.ld_o, a.dO, a.ld_do = o.data_ptr(), o.stride(0), do.data_ptr(), do.stride(0)
    a.lse, a.delta = lse.data_ptr(), delta.data_ptr()
    a.dQ = dqkv.data_ptr()
    a.dK = dqkv.data_ptr() + inner * 2
    a.dV = dqkv.data_ptr() + 2 * inner * 2
    a.ld_dqkv = dqkv.stride(0)
    a.seg_start, a.nseg = seg_start.data_ptr(), nseg
    a.rows, a.H, a.hd, a.scale = rows, heads, head_dim, scale
    a.status = _lib.status_word(q.device).data_ptr()
    a.max_tiles = -(-rows // 128) + nseg
    L = _lib.lib()
    L.nb_flash_bwd.argtypes = [C.POINTER(_lib.FlashBwdArgs), C.c_void_p]
    L.nb_flash_bwd.restype = C.c_int
    rc = L.nb_flash_bwd(C.byref(a), C.c_void_p(_lib.stream_ptr()))
    if rc != 0:
        raise RuntimeError(f"nb_flash_bwd failed with code {rc}")
    _lib.count_launch(3)
    return dqkv
