"""Python front end of the persistent tcgen05 grouped GEMM (``csrc/gemm.cu``).

``gemm_rows``: ``C[r] = A[r] . B[group(r)]`` for rows packed by group (forward and data
gradients). ``gemm_reduce``: ``C[g] (+)= A[rows of g]^T . B[rows of g]`` (weight
gradients). Operands are bf16; "MN-major" means the operand is stored with its M (or N)
index contiguous, i.e. as the transpose of the usual row-of-K layout — both are read by
TMA without any copy.
"""

from __future__ import annotations

import ctypes as C
import dataclasses
import os

import torch
from torch import Tensor

from nestor_b200.ops import _lib

STORE_BF16, STORE_F32, ACCUM_F32, SWIGLU, SWIGLU_BWD, STORE_BF16_STATS, AXPBY_BF16 = range(7)
# STORE_BF16_STATS writes this many (max, sum-exp) partials per row and n-tile: extra_out[0] is [rows, n_tiles * STATS_PARTS, 2]
STATS_PARTS = 2

# Producer tuning (see csrc/gemm.cu): L2 look-ahead in k-blocks (off: measured slower, the TMA issue rate is the
# limit, not DRAM latency), and a cap on pipeline stages (0 = all that fit).
PREFETCH_DIST = int(os.environ.get("NESTOR_B200_GEMM_PREFETCH", "0"))
MAX_STAGES = int(os.environ.get("NESTOR_B200_GEMM_STAGES", "0"))
# bf16 outputs of row-grouped products leave as tiled (TMA) stores where a warp's 32 rows are whole; "0" keeps the
# row-masked vector stores everywhere
TILED_STORE = os.environ.get("NESTOR_B200_TILED_STORE", "1") == "1"
# weight-gradient (reduction-grouped) products on CTA pairs: "auto", "1" or "0"
REDUCE_PAIR = os.environ.get("NESTOR_B200_REDUCE_PAIR", "auto")
# CTA pairs: 256-row tiles where each CTA of a 2-CTA cluster stages half of B (cta_group::2 MMAs). The L2 -> SM
# traffic per FLOP drops by the B half, which is what bounds these shapes. "auto" uses pairs for big row counts.
PAIR = os.environ.get("NESTOR_B200_GEMM_PAIR", "auto")
_PAIR_MIN_ROWS = 4096
DEBUG = 0   # kernel timing experiments (see csrc/gemm.cu); never set outside of them
_L2_RESIDENT_BYTES = 48 << 20    # a shared B operand smaller than this stays in L2 without help


@dataclasses.dataclass
class Gather:
    """Where a rank-sharded weight operand lives, for the all-gather fused into ``gemm_rows``.

    ``src[r]`` is the address of rank ``r``'s weight arena as mapped into this process and ``arena_ptr`` the
    address of the local one: the operand handed to ``gemm_rows`` is a view of the local arena and only tells
    *where* in an arena the groups sit; their values are read from each group's owner (``group // groups_per_rank``)
    into ``stage`` by a copy warp in every CTA of the same launch, and the tensor maps of the product point at
    ``stage``. ``lanes`` lanes of that warp copy independently; ``chunk`` x ``nbuf`` x ``lanes`` bytes of shared
    memory per CTA go to the copy rings (``nbuf * lanes <= 8``).
    ``flags`` is an ``int32`` tensor of at least ``groups + 1`` zeros shared by stream-ordered launches. Every CTA of a
    gathering launch must be resident at once (the launcher clamps the grid to what the occupancy calculator grants);
    do not run it next to another kernel that holds SMs for its whole duration.
    """

    src: list[int]
    arena_ptr: int
    stage: Tensor
    flags: Tensor
    groups_per_rank: int
    chunk: int = 8192
    nbuf: int = 4
    lanes: int = 1
    wait_polls: int = 0      # polls (>= 100 ns each) a B producer waits for a group's chunks; 0 = about half a second


def pick_bn(n: int, *, mult: int = 16, cap: int = 256) -> int:
    """Tile width: least padded-N plus a fixed cost per tile, ties to the wider tile; multiples of ``mult`` up to ``cap``.

    The fixed cost stands for what a tile costs beyond its columns (operand A fetched again, MMA issue and hand-over
    latency). For MN-major B (``mult`` 64) it is large: on ``[98304 x 216] x [64, 216, 640]`` three tiles of 256 columns
    ran in 56 us against 68 us for five tiles of 128, although a sixth of the wide tiles' columns is padding.
    """

    fixed = 160.0 if mult >= 64 else 24.0
    best, best_cost = mult, None
    for bn in range(mult, cap + 1, mult):
        tiles = -(-n // bn)
        cost = tiles * (bn + fixed)
        if best_cost is None or cost <= best_cost:
            best, best_cost = bn, cost
    return best


def rows_buffer(rows: int, cols: int, dtype: torch.dtype = torch.bfloat16, device=None) -> Tensor:
    """``[rows, cols]`` activation buffer whose row pitch is a multiple of 64 elements.

    The weight-gradient product reads activations "MN-major" (as ``[k rows, M or N columns]``); with a pitch
    that covers whole 64-column atoms the kernel fetches every atom of a pipeline stage with one TMA
    instruction. The padding columns are never written and only ever reach masked outputs.
    """

    pitch = -(-cols // 64) * 64
    buf = torch.empty(rows, pitch, dtype=dtype, device=device)
    return buf if pitch == cols else buf[:, :cols]


def _operand(t: Tensor | None, *, grouped: bool) -> _lib.Operand:
    if t is None:
        return _lib.Operand(None, 0, 0, 0, 0, 0)
    assert t.dtype == torch.bfloat16 and t.stride(-1) == 1, "operands are bf16 with a contiguous last dim"
    assert t.data_ptr() % 16 == 0 and (t.stride(-2) * 2) % 16 == 0, "TMA needs 16-byte aligned base and row pitch"
    if t.ndim == 3:
        assert (t.stride(0) * 2) % 16 == 0
        return _lib.Operand(t.data_ptr(), t.shape[1], t.shape[2], t.stride(1), t.shape[0], t.stride(0))
    return _lib.Operand(t.data_ptr(), t.shape[0], t.shape[1], t.stride(0), 1, t.shape[0] * t.stride(0))


def _stage_for_gather(a: _lib.GemmArgs, g: Gather, B: Tensor, B2: Tensor | None) -> tuple[Tensor, Tensor | None]:
    """Fill the gather fields of ``a`` and return the staged stand-ins of ``B`` / ``B2`` (dense, same shapes)."""

    assert B.ndim == 3 and B[0].is_contiguous() and (B2 is None or (B2.shape == B.shape and B2.stride() == B.stride()))
    groups, group_elems = B.shape[0], B.shape[1] * B.shape[2]
    assert groups % g.groups_per_rank == 0 and groups // g.groups_per_rank <= len(g.src)
    assert (group_elems * 2) % 16 == 0 and (B.stride(0) * 2) % 16 == 0 and g.stage.data_ptr() % 256 == 0
    segs = [B] if B2 is None else [B, B2]
    assert g.stage.numel() * g.stage.element_size() >= len(segs) * groups * group_elems * 2, "staging buffer too small"
    assert g.flags.numel() >= groups + 1 and g.flags.dtype == torch.int32
    flat = g.stage.view(torch.bfloat16).view(-1)
    staged = []
    for i, t in enumerate(segs):
        a.gather_seg_src_off[i] = t.data_ptr() - g.arena_ptr
        a.gather_seg_dst_off[i] = i * groups * group_elems * 2
        staged.append(flat[i * groups * group_elems : (i + 1) * groups * group_elems].view(B.shape))
    for r, ptr in enumerate(g.src):
        a.gather_src[r] = ptr
    a.gather_dst = g.stage.data_ptr()
    a.gather_group_bytes, a.gather_group_stride_src = group_elems * 2, B.stride(0) * 2
    a.gather_nseg, a.gather_groups_per_rank, a.gather_on, a.gather_chunk = len(segs), g.groups_per_rank, 1, g.chunk
    a.gather_nbuf, a.gather_lanes = g.nbuf, g.lanes
    a.gather_wait_polls = int(g.wait_polls)
    a.gather_flags = g.flags.data_ptr()
    return staged[0], (staged[1] if B2 is not None else None)


def _launch(args: _lib.GemmArgs) -> None:
    rc = _lib.lib().nb_gemm(C.byref(args), C.c_void_p(_lib.stream_ptr()))
    if rc != 0:
        raise RuntimeError(f"nb_gemm failed with code {rc}")
    _lib.count_launch()


def gemm_rows(A: Tensor, B: Tensor, *, offsets: Tensor | None = None, groups: int = 1, b_mn: bool = False,
              out: Tensor | None = None, epilogue: int = STORE_BF16, alpha: float = 1.0, beta: float = 0.0,
              bn: int | None = None,
              A2: Tensor | None = None, B2: Tensor | None = None, extra_out: tuple = (), extra_in: tuple = (),
              n: int | None = None, n_valid: int = 0, sms: int = 0, trace: Tensor | None = None,
              pair: bool | None = None, gather: Gather | None = None) -> Tensor:
    """Row-grouped GEMM.

    ``A [rows, K]``; ``B`` is ``[G, N, K]`` (K-major) or ``[G, K, N]`` (``b_mn``) — 2-D for a
    single shared matrix. ``offsets [G+1]`` (int32, device) bound the groups; ``None`` with
    ``groups == 1`` means one group over all rows. ``A2/B2`` extend the reduction. With
    ``epilogue == SWIGLU``, ``B`` is the gate bank and ``B2`` the up bank (both ``[G, K, h]``);
    ``out`` receives ``silu(gate) * up`` and ``extra_out = (gate, up)``. With ``epilogue == AXPBY_BF16`` the
    result is ``alpha * (A . B) + beta * extra_in[0]`` (bf16, same shape and pitch rules as ``out``). With ``gather``, ``B`` (and ``B2``)
    are 3-D views of the local weight arena whose groups are owned by different ranks: the launch stages them
    from their owners while it computes (see ``Gather``).
    """

    rows, K = A.shape
    if b_mn:
        N = B.shape[-1] if n is None else n
    else:
        N = B.shape[-2] if n is None else n
    swiglu = epilogue == SWIGLU
    if swiglu:
        N = 2 * B.shape[-1]
    if pair is None:
        # pairs pay off when the main loop dominates (long K) and the tile is wide; short-K products are bound by
        # the epilogue, where 256-row tiles only add masked rows at group ends
        wide = swiglu or (bn or (N if b_mn else pick_bn(N))) >= 192
        pair = PAIR == "1" or (PAIR == "auto" and rows >= _PAIR_MIN_ROWS and K >= 512 and wide and (not b_mn or swiglu or N >= 256))
    if bn is None:
        if pair:
            bn = 256 if swiglu else pick_bn(N, mult=128 if b_mn else 16)
        else:
            bn = 128 if swiglu else pick_bn(N, mult=64 if b_mn else 16)
    if pair and (bn % 16 or (b_mn and bn % 128)):
        pair = False
        if swiglu:
            bn = 128
    dev = A.device
    if out is None:
        dt = torch.float32 if epilogue in (STORE_F32, ACCUM_F32) else torch.bfloat16
        out = torch.empty(rows, N // 2 if swiglu else N, dtype=dt, device=dev)
    # vector stores of the epilogue: 16-byte aligned rows, widths in whole 8-column (bf16) / 4-column (fp32) groups
    per16 = 16 // out.element_size()
    assert out.stride(-1) == 1 and out.stride(0) % per16 == 0 and out.data_ptr() % 16 == 0, "misaligned GEMM output"
    assert (N // 2 if swiglu else N) % per16 == 0, f"GEMM output width {N} must be a multiple of {per16}"
    a = _lib.GemmArgs()
    a.mode, a.groups, a.BN, a.epilogue = 0, groups, bn, epilogue
    a.M, a.N, a.K, a.K2 = rows, N, K, (A2.shape[1] if A2 is not None else 0)
    a.offsets = offsets.data_ptr() if offsets is not None else None
    a.rows_per_group = rows if offsets is None else 0
    if offsets is None and groups != 1:
        assert rows % groups == 0
        a.rows_per_group = rows // groups
    a.a_mn, a.b_mn, a.b_grouped = 0, int(b_mn), int(B.ndim == 3)
    if gather is not None:
        B, B2 = _stage_for_gather(a, gather, B, B2)
    a.A, a.B = _operand(A, grouped=False), _operand(B, grouped=True)
    a.A2, a.B2 = _operand(A2, grouped=False), _operand(B2, grouped=True)
    a.C, a.ldc, a.c_group_stride = out.data_ptr(), out.stride(0), 0
    a.C2 = extra_out[0].data_ptr() if len(extra_out) > 0 else None
    a.C3 = extra_out[1].data_ptr() if len(extra_out) > 1 else None
    a.E1 = extra_in[0].data_ptr() if len(extra_in) > 0 else None
    a.E2 = extra_in[1].data_ptr() if len(extra_in) > 1 else None
    a.lde = extra_in[0].stride(0) if len(extra_in) > 0 else 0
    a.alpha, a.beta = alpha, beta
    a.n_valid = n_valid
    a.status = _lib.status_word(dev).data_ptr()
    a.pair = int(pair)
    a.debug = DEBUG
    a.no_tiled_store = 0 if TILED_STORE else 1
    a.max_m_tiles = -(-rows // (256 if pair else 128)) + groups
    a.sms = sms
    a.trace = trace.data_ptr() if trace is not None else None
    # A is streamed once per n-tile pass; B (weights) is re-read by every m-tile and only needs help when it is large
    a.prefetch_dist, a.max_stages = PREFETCH_DIST, MAX_STAGES
    a.prefetch_ops = 1 | (2 if B.numel() * 2 > _L2_RESIDENT_BYTES else 0)
    _launch(a)
    return out


def gemm_reduce(A: Tensor, B: Tensor, *, offsets: Tensor | None = None, groups: int = 1, out: Tensor,
                epilogue: int = ACCUM_F32, alpha: float = 1.0, bn: int | None = None, sms: int = 0,
                trace: Tensor | None = None, pair: bool | None = None) -> Tensor:
    """Reduction-grouped GEMM: ``out[g] (+)= A[rows_g]^T @ B[rows_g]`` with ``A [rows, M]``, ``B [rows, N]``.

    ``out`` is ``[G, M, N]`` (or ``[M, N]`` for one group) with a contiguous last dim; fp32 for the
    store/accumulate epilogues.
    """

    rows, M = A.shape
    N = B.shape[1]
    assert B.shape[0] == rows
    if bn is None:
        bn = pick_bn(N, mult=64)
    a = _lib.GemmArgs()
    a.mode, a.groups, a.BN, a.epilogue = 1, groups, bn, epilogue
    a.M, a.N, a.K, a.K2 = M, N, rows, 0
    a.offsets = offsets.data_ptr() if offsets is not None else None
    a.rows_per_group = 0 if offsets is not None else rows // groups
    a.a_mn, a.b_mn, a.b_grouped = 1, 1, 0
    a.A, a.B = _operand(A, grouped=False), _operand(B, grouped=False)
    a.A2, a.B2 = _operand(None, grouped=False), _operand(None, grouped=False)
    o3 = out if out.ndim == 3 else out.unsqueeze(0)
    assert o3.stride(-1) == 1
    per16 = 16 // out.element_size()
    assert o3.stride(1) % per16 == 0 and o3.stride(0) % per16 == 0 and out.data_ptr() % 16 == 0 and N % per16 == 0, \
        "weight-gradient output rows must be 16-byte aligned (pad the inner dim)"
    a.C, a.ldc, a.c_group_stride = o3.data_ptr(), o3.stride(1), o3.stride(0)
    a.alpha = alpha
    if pair is None:
        # a CTA pair (256 x bn tile, each CTA staging its 128 A columns and half of B) moves a third less data into
        # each SM per FLOP; it needs B halves of whole 64-column atoms and more than one 128-row tile of work
        pair = REDUCE_PAIR == "1" or (REDUCE_PAIR == "auto" and bn % 128 == 0 and M > 128)
    if pair and bn % 128:
        pair = False
    a.pair = int(pair)
    # few output tiles and a long reduction: let several CTAs share a tile (fp32 atomic adds)
    tiles = groups * -(-M // (256 if pair else 128)) * -(-N // bn) * (2 if pair else 1)
    kblocks = max(1, rows // (64 * groups))
    a.splits = 1
    if epilogue == ACCUM_F32 and tiles < (_lib.sm_count(A.device) * 13) // 16:
        a.splits = max(1, min(_lib.sm_count(A.device) // tiles, kblocks // 4))
    a.status = _lib.status_word(A.device).data_ptr()
    a.max_m_tiles = 0
    a.sms = sms
    a.prefetch_dist, a.max_stages, a.prefetch_ops = PREFETCH_DIST, MAX_STAGES, 3
    a.trace = trace.data_ptr() if trace is not None else None
    a.debug = DEBUG
    a.no_tiled_store = 0 if TILED_STORE else 1
    _launch(a)
    return out
