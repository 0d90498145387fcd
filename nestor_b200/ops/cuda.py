"""Kernel-backed bodies of the hot ops (CUDA tensors only).

Each op is a ``torch.autograd.Function`` whose forward and backward are sequences of
launches from the in-tree sm_100a library: the persistent tcgen05 grouped GEMM
(:mod:`nestor_b200.ops.gemm`), the varlen flash-attention kernels
(:mod:`nestor_b200.ops.flash`) and the gather / combine / RoPE / cross-entropy / depth-read
kernels of ``csrc/pointwise.cu``. Signatures match :mod:`nestor_b200.ops.reference`.

Weight gradients: when a weight operand comes from the parameter arena it carries
``_nb_grad`` (its fp32 gradient view) and the reduction-grouped GEMM accumulates into that
view directly; autograd then sees ``None`` for the operand. Otherwise an fp32 gradient
tensor is returned through autograd as usual.
"""

from __future__ import annotations

import ctypes as C
import math
import os

import torch
from torch import Tensor

from nestor_b200.ops import _lib, flash, gemm as G
from nestor_b200.ops import reference as ref

# Shapes beyond a kernel's built-in limits run the PyTorch statement of the op instead. That is never silent: the first
# such call of each kind warns with the limit it crossed, every call is counted (``oracle_path_report()``), and
# ``NESTOR_B200_STRICT=1`` turns it into an error.
_oracle_calls: dict[str, int] = {}


def _oracle_path(op: str, why: str) -> None:
    import os
    import warnings
    if os.environ.get("NESTOR_B200_STRICT", "0") == "1":
        raise RuntimeError(f"{op}: {why}; the kernel library has no body for this shape (NESTOR_B200_STRICT=1)")
    if op not in _oracle_calls:
        warnings.warn(f"{op}: {why}; running the PyTorch statement of the op instead of the sm_100a kernel", RuntimeWarning,
                      stacklevel=3)
    _oracle_calls[op] = _oracle_calls.get(op, 0) + 1


def note_eager(op: str) -> None:
    """Count a call of an op that has no fused kernel (a model option outside the registered cells runs it as plain
    PyTorch arithmetic on the GPU by design: no warning, but it shows in the report)."""

    _oracle_calls[op] = _oracle_calls.get(op, 0) + 1


def oracle_path_report() -> dict[str, int]:
    """How many calls of each op ran as PyTorch statements on CUDA tensors since import: shapes or options beyond a
    kernel's limits, and ops without a fused kernel."""

    return dict(_oracle_calls)
from nestor_b200.ops.reference import ColumnPlan, ExpertPlan

BF16 = torch.bfloat16
_protos_done = False


def _L():
    global _protos_done
    L = _lib.lib()
    if not _protos_done:
        vp, i, l, f = C.c_void_p, C.c_int, C.c_long, C.c_float
        L.nb_gather_rows.argtypes = [vp, i, l, vp, i, vp, l, i, i, l, vp]
        L.nb_combine_rows.argtypes = [vp, l, vp, vp, i, vp, l, i, i, i, i, l, i, vp]
        L.nb_combine_bwd.argtypes = [vp, l, vp, l, vp, vp, i, vp, l, vp, i, i, vp, vp, l, i, f, l, vp]
        L.nb_rope.argtypes = [vp, l, vp, i, i, i, i, f, f, vp]
        L.nb_repack_heads.argtypes = [vp, l, vp, l, i, i, i, i, i, vp]
        L.nb_repack_heads.restype = C.c_int
        L.nb_ce_grad.argtypes = [vp, l, i, vp, i, vp, l, vp, i, vp]
        L.nb_depth_read_norm.argtypes = [vp, i, vp, vp, vp, f, f, vp, vp, vp, vp, i, i, vp]
        L.nb_depth_read_norm_bwd.argtypes = [vp, vp, i, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i, i, C.c_ulonglong, vp, vp, vp]
        L.nb_depth_read_norm_bwd.restype = C.c_int
        L.nb_mid_source.argtypes = [vp, vp, vp, i, i, i, vp]
        L.nb_layer_combine.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, i, i, i, vp]
        L.nb_layer_combine_bwd.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, i, i, i, vp]
        L.nb_block_exit.argtypes = [vp, vp, vp, i, i, i, vp]
        L.nb_block_exit_bwd.argtypes = [vp, vp, vp, i, i, i, vp]
        for fn in (L.nb_mid_source, L.nb_layer_combine, L.nb_layer_combine_bwd, L.nb_block_exit, L.nb_block_exit_bwd):
            fn.restype = C.c_int
        L.nb_expert_plan.argtypes = [vp, i, i, vp, vp, vp, vp, vp]
        L.nb_column_plan.argtypes = [vp, i, i, i, i, i, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp]
        L.nb_column_plan.restype = C.c_int
        L.nb_route_fwd.argtypes = [vp, vp]
        L.nb_route_bwd.argtypes = [vp, vp, vp, vp, l, i, vp, vp]
        for fn in (L.nb_expert_plan, L.nb_route_fwd, L.nb_route_bwd):
            fn.restype = C.c_int
        L.nb_ns_prepare.argtypes = [vp, vp, i, i, i, i, i, vp, vp]
        L.nb_ns_finish.argtypes = [vp, vp, i, i, i, i, i, vp]
        L.nb_ns_prepare.restype = L.nb_ns_finish.restype = C.c_int
        for fn in (L.nb_gather_rows, L.nb_combine_rows, L.nb_combine_bwd, L.nb_rope, L.nb_ce_grad,
                   L.nb_depth_read_norm):
            fn.restype = C.c_int
        _protos_done = True
    return L


def _ck(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")
    _lib.count_launch()


def bounds_check_report() -> dict | None:
    """First index violation the gather-style kernels recorded since the last call (checking library builds only:
    ``NESTOR_B200_BOUNDS_CHECK=1``); ``None`` when there was none. Synchronises the device."""

    L = _L()
    if not L.nb_bounds_check_enabled():
        return None
    rec = (C.c_int * 4)()
    rc = L.nb_bounds_check_read(rec)
    if rc != 0:
        raise RuntimeError(f"nb_bounds_check_read failed with code {rc}")
    if rec[0] == 0:
        return None
    return {"code": rec[0], "kernel": {1: "gather_rows", 2: "combine_rows", 3: "combine_bwd"}.get(rec[1], rec[1]),
            "index": rec[2], "row": rec[3]}


def _ptr(t: Tensor | None):
    return None if t is None else t.data_ptr()


def _st():
    return C.c_void_p(_lib.stream_ptr())


# ------------------------------------------------------------------- pointwise launchers
def gather_rows(src: Tensor, idx: Tensor, div: int = 1) -> Tensor:
    """``out[r] = bf16(src[idx[r] // div])`` for a 2-D fp32/bf16 ``src`` with contiguous rows."""

    rows, d = idx.numel(), src.shape[-1]
    out = torch.empty(rows, d, dtype=BF16, device=src.device)
    _ck(_L().nb_gather_rows(src.data_ptr(), int(src.dtype == torch.float32), src.stride(0), idx.data_ptr(), div,
                            out.data_ptr(), d, rows, d, src.shape[0], _st()), "gather_rows")
    return out


def combine_rows(y: Tensor, idx: Tensor, w: Tensor | None, group: int, n_out: int, out: Tensor | None = None,
                 accumulate: bool = False, round_products: bool = True, out_dtype: torch.dtype = torch.float32) -> Tensor:
    """``out[o] = sum_{e<group} y[idx[o*group+e]] * w[o*group+e]`` in fp32 (each product first rounded to
    bf16 when ``round_products``); ``out_dtype=bfloat16`` stores the fp32 sums rounded once (no separate cast pass)."""

    d = y.shape[-1]
    if out is None:
        out = torch.empty(n_out, d, dtype=out_dtype, device=y.device)
    assert out.dtype in (torch.float32, BF16) and not (out.dtype == BF16 and accumulate)
    _ck(_L().nb_combine_rows(y.data_ptr(), y.stride(0), idx.data_ptr(), _ptr(w), group, out.data_ptr(), out.stride(0),
                             n_out, d, int(accumulate), int(round_products), y.shape[0], int(out.dtype == BF16), _st()),
        "combine_rows")
    return out


def combine_bwd(g: Tensor, y: Tensor, slot_of_row: Tensor, w: Tensor | None, group: int,
                need_dw: bool, shared: tuple = (), shared_div: int = 1,
                shared_scale: float = 1.0) -> tuple[Tensor, Tensor | None]:
    """Backward of ``combine_rows``. ``shared`` holds up to two ``[n, d]`` fp32 tensors: extra gradients of the
    combined output that ``shared_div`` consecutive slots have in common, added as
    ``shared[i][slot // shared_div] * shared_scale``."""

    shared = [t for t in shared if t is not None]
    sh0 = shared[0] if len(shared) > 0 else None
    sh1 = shared[1] if len(shared) > 1 else None
    assert sh1 is None or sh1.stride(0) == sh0.stride(0)

    rows, d = y.shape
    dy = torch.empty(rows, d, dtype=BF16, device=y.device)
    dw = torch.empty(rows, dtype=torch.float32, device=y.device) if need_dw else None
    _ck(_L().nb_combine_bwd(g.data_ptr(), g.stride(0), y.data_ptr(), y.stride(0), slot_of_row.data_ptr(), _ptr(w), group,
                            dy.data_ptr(), d, _ptr(dw), rows, d, _ptr(sh0), _ptr(sh1), sh0.stride(0) if sh0 is not None else 0,
                            shared_div, float(shared_scale), g.shape[0] * group, _st()), "combine_bwd")
    return dy, dw


def rope_(buf: Tensor, pos: Tensor, heads: int, head_dim: int, k_offset: int, base: float, sign: float) -> None:
    """In-place RoPE on the q (columns 0..) and k (columns ``k_offset``..) ranges of ``buf``."""

    _ck(_L().nb_rope(buf.data_ptr(), buf.stride(0), pos.data_ptr(), buf.shape[0], heads, head_dim, k_offset,
                     float(base), float(sign), _st()), "rope")


def repack_heads(src: Tensor, nheads: int, hs: int, hd: int, dst_cols: int) -> Tensor:
    """``[rows, nheads*hs]`` -> ``[rows, dst_cols]`` with head stride ``hd`` (zero-filled padding, or padding stripped)."""

    rows = src.shape[0]
    dst = G.rows_buffer(rows, dst_cols, BF16, src.device)
    _ck(_L().nb_repack_heads(src.data_ptr(), src.stride(0), dst.data_ptr(), dst.stride(0), rows, nheads, hs, hd, dst_cols,
                             _st()), "repack_heads")
    return dst


def _wgrad(a: Tensor, b: Tensor, w: Tensor, *, offsets: Tensor | None, groups: int, transpose_out: bool = False):
    """Weight gradient ``a^T @ b`` per group. Accumulates into ``w._nb_grad`` when present (returns None)."""

    target = getattr(w, "_nb_grad", None)
    if target is not None:
        G.gemm_reduce(a, b, offsets=offsets, groups=groups, out=target, epilogue=G.ACCUM_F32)
        return None
    shape = (groups, a.shape[1], b.shape[1]) if w.ndim == 3 else (a.shape[1], b.shape[1])
    out = torch.empty(shape, dtype=torch.float32, device=a.device)
    G.gemm_reduce(a, b, offsets=offsets, groups=groups, out=out, epilogue=G.STORE_F32)
    return out.to(w.dtype)


# ---------------------------------------------------------------------------- linear
class _Linear(torch.autograd.Function):
    """``y = x @ w^T`` with ``w [N, K]`` (bf16). ``x`` may be fp32 (rounded to bf16 on the way in)."""

    @staticmethod
    def forward(ctx, x: Tensor, w: Tensor) -> Tensor:
        xb = x if x.dtype == BF16 else x.to(BF16)
        n = w.shape[0]
        npad = max(8, -(-n // 8) * 8)
        y = G.gemm_rows(xb.contiguous(), w, n=npad)
        ctx.save_for_backward(xb, w)
        ctx.n, ctx.x_dtype = n, x.dtype
        ctx.w_ref = w
        return y if npad == n else y[:, :n]

    @staticmethod
    def backward(ctx, dy: Tensor):
        xb, w = ctx.saved_tensors
        n = ctx.n
        npad = max(8, -(-n // 8) * 8)
        dyb = dy.to(BF16)
        if npad != n:
            dyb = torch.nn.functional.pad(dyb, (0, npad - n))
        dyb = dyb.contiguous()
        dx = None
        if ctx.needs_input_grad[0]:
            dx = G.gemm_rows(dyb, w, b_mn=True, n=w.shape[1]).to(ctx.x_dtype)   # w as [K=N, N=d] MN-major
        dw = None
        if ctx.needs_input_grad[1]:
            wv = ctx.w_ref
            target = getattr(wv, "_nb_grad", None)
            if target is not None and npad == n:
                G.gemm_reduce(dyb, xb, out=target, epilogue=G.ACCUM_F32)
            else:
                full = torch.empty(npad, xb.shape[1], dtype=torch.float32, device=xb.device)
                G.gemm_reduce(dyb, xb, out=full, epilogue=G.STORE_F32)
                if target is not None:
                    target.add_(full[:n])
                else:
                    dw = full[:n].to(w.dtype)
        return dx, dw


def linear(x: Tensor, w: Tensor) -> Tensor:
    return _Linear.apply(x, w)


def router_scores(x: Tensor, w1: Tensor | None, w2: Tensor, cd: torch.dtype) -> Tensor:
    h = x
    if w1 is not None:
        h = torch.nn.functional.gelu(linear(h, w1.to(BF16) if w1.dtype != BF16 else w1))
    return linear(h, w2.to(BF16) if w2.dtype != BF16 else w2)


# ----------------------------------------------------------------------- expert bank
# Set by the trainer when expert banks are rank-sharded (parallel/shard.py: ShardedBanks): the bank products then
# stage their weights from the owners' arenas inside the GEMM launch instead of reading the local copy.
BANK_SHARDS = None


def _bank_gather(w, w2=None):
    return BANK_SHARDS.spec(w, w2) if BANK_SHARDS is not None else None


class _ExpertBank(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weights, w_up, w_gate, w_down, plan: ExpertPlan, group: int):
        T, d = x.shape
        E, _, h = w_up.shape
        xs = gather_rows(x, plan.order, div=plan.slots)                       # dispatch gather [n, d]
        hh, gt, ut = (G.rows_buffer(plan.n, h, BF16, x.device) for _ in range(3))
        G.gemm_rows(xs, w_gate, B2=w_up, offsets=plan.offsets, groups=E, b_mn=True, out=hh, epilogue=G.SWIGLU,
                    extra_out=(gt, ut), gather=_bank_gather(w_gate, w_up))
        y = G.gemm_rows(hh, w_down, offsets=plan.offsets, groups=E, b_mn=True, gather=_bank_gather(w_down))  # [n, d]
        wf = weights.float().contiguous().view(-1)
        out = combine_rows(y, plan.inv, wf, group, T * (plan.slots // group))
        ctx.save_for_backward(xs, hh, gt, ut, y, wf, w_up, w_gate, w_down)
        ctx.plan, ctx.group, ctx.T, ctx.x_dtype, ctx.w_dtype = plan, group, T, x.dtype, weights.dtype
        ctx.w_refs = (w_up, w_gate, w_down)
        return out.view(T, plan.slots // group, d)

    @staticmethod
    def backward(ctx, dout):
        xs, hh, gt, ut, y, wf, w_up, w_gate, w_down = ctx.saved_tensors
        plan, group, T = ctx.plan, ctx.group, ctx.T
        E, d, h = w_up.shape
        g2 = dout.contiguous().view(-1, d).float()
        dy, dw_sorted = combine_bwd(g2, y, plan.order, wf, group, need_dw=ctx.needs_input_grad[1])
        dgt, dut = G.rows_buffer(plan.n, h, BF16, dy.device), G.rows_buffer(plan.n, h, BF16, dy.device)
        # dH = dY . Wd^T fused with the SwiGLU derivative; Wd [E, h, d] is the K-major B of this product
        G.gemm_rows(dy, w_down, offsets=plan.offsets, groups=E, out=dgt, epilogue=G.SWIGLU_BWD, extra_out=(dut,),
                    extra_in=(gt, ut), gather=_bank_gather(w_down))
        dx = None
        if ctx.needs_input_grad[0]:
            dxs = G.gemm_rows(dgt, w_gate, A2=dut, B2=w_up, offsets=plan.offsets, groups=E,
                              gather=_bank_gather(w_gate, w_up))                                # [n, d]
            direct = ctx.x_dtype in (torch.float32, BF16)
            dx = combine_rows(dxs, plan.inv, None, plan.slots, T, out_dtype=ctx.x_dtype if direct else torch.float32)
            dx = dx if direct else dx.to(ctx.x_dtype)
        dweights = None
        if dw_sorted is not None:      # the kernel indexes dw by flat slot already
            dweights = dw_sorted.view(T, plan.slots).to(ctx.w_dtype)
        wu, wg, wd = ctx.w_refs
        d_down = _wgrad(hh, dy, wd, offsets=plan.offsets, groups=E) if ctx.needs_input_grad[4] else None
        d_gate = _wgrad(xs, dgt, wg, offsets=plan.offsets, groups=E) if ctx.needs_input_grad[3] else None
        d_up = _wgrad(xs, dut, wu, offsets=plan.offsets, groups=E) if ctx.needs_input_grad[2] else None
        return dx, dweights, d_up, d_gate, d_down, None, None


class _PointwiseBank(torch.autograd.Function):
    """Routed bank of pointwise experts ``down(act(up(x)))``: the same dispatch gather, grouped products and weighted
    combine as the SwiGLU bank, with the activation (and its derivative) as one elementwise pass between the two
    products instead of a fused epilogue."""

    @staticmethod
    def forward(ctx, x, weights, w_up, w_down, plan: ExpertPlan, group: int, activation: str):
        T, d = x.shape
        E, _, h = w_up.shape
        act = ref.POINTWISE_ACTIVATIONS[activation]
        xs = gather_rows(x, plan.order, div=plan.slots)                       # dispatch gather [n, d]
        # the up product reads its bank K-major ([E, h, d]); the transposed copy is per call and bank-sized
        u = G.gemm_rows(xs, w_up.transpose(1, 2).contiguous(), offsets=plan.offsets, groups=E)      # [n, h]
        a = G.rows_buffer(plan.n, h, BF16, x.device)
        a.copy_(act(u))
        y = G.gemm_rows(a, w_down, offsets=plan.offsets, groups=E, b_mn=True)                        # [n, d]
        wf = weights.float().contiguous().view(-1)
        out = combine_rows(y, plan.inv, wf, group, T * (plan.slots // group))
        ctx.save_for_backward(xs, u, a, y, wf, w_up, w_down)
        ctx.plan, ctx.group, ctx.T, ctx.x_dtype, ctx.w_dtype, ctx.act = plan, group, T, x.dtype, weights.dtype, act
        ctx.w_refs = (w_up, w_down)
        return out.view(T, plan.slots // group, d)

    @staticmethod
    def backward(ctx, dout):
        xs, u, a, y, wf, w_up, w_down = ctx.saved_tensors
        plan, group, T = ctx.plan, ctx.group, ctx.T
        E, d, h = w_up.shape
        g2 = dout.contiguous().view(-1, d).float()
        dy, dw_sorted = combine_bwd(g2, y, plan.order, wf, group, need_dw=ctx.needs_input_grad[1])
        da = G.gemm_rows(dy, w_down, offsets=plan.offsets, groups=E)            # dA = dY . Wd^T, Wd [E, h, d] K-major
        with torch.enable_grad():
            u32 = u.float().requires_grad_(True)
            slope = torch.autograd.grad(ctx.act(u32), u32, da.float())[0]
        du = G.rows_buffer(plan.n, h, BF16, dy.device)
        du.copy_(slope)
        dx = None
        if ctx.needs_input_grad[0]:
            dxs = G.gemm_rows(du, w_up, offsets=plan.offsets, groups=E)                             # [n, d]
            direct = ctx.x_dtype in (torch.float32, BF16)
            dx = combine_rows(dxs, plan.inv, None, plan.slots, T, out_dtype=ctx.x_dtype if direct else torch.float32)
            dx = dx if direct else dx.to(ctx.x_dtype)
        dweights = None
        if dw_sorted is not None:
            dweights = dw_sorted.view(T, plan.slots).to(ctx.w_dtype)
        wu, wd = ctx.w_refs
        d_down = _wgrad(a, dy, wd, offsets=plan.offsets, groups=E) if ctx.needs_input_grad[3] else None
        d_up = _wgrad(xs, du, wu, offsets=plan.offsets, groups=E) if ctx.needs_input_grad[2] else None
        return dx, dweights, d_up, d_down, None, None, None


POINTWISE_BANK_KERNELS = os.environ.get("NESTOR_B200_POINTWISE_BANK", "1") == "1"


def expert_bank(x, plan, weights, w_up, w_gate, w_down, cd, group, activation="swiglu"):
    if activation != "swiglu":
        if POINTWISE_BANK_KERNELS and BANK_SHARDS is None:
            return _PointwiseBank.apply(x, weights, w_up, w_down, plan, group, activation)
        # (rank-sharded banks stage their weights inside the SwiGLU launches only)
        _oracle_path("expert_bank", f"pointwise activation {activation!r}")
        return ref.expert_bank(x, plan, weights, w_up, None, w_down, cd, group, activation)
    return _ExpertBank.apply(x, weights, w_up, w_gate, w_down, plan, group)


def dense_swiglu(x, w_up, w_gate, w_down, cd, activation="swiglu"):
    u = linear(x, w_up)
    if activation != "swiglu":
        return linear(ref.POINTWISE_ACTIVATIONS[activation](u), w_down).float()
    g = linear(x, w_gate)
    return linear(torch.nn.functional.silu(g) * u, w_down).float()


# ------------------------------------------------------------------------- attention
class _MidState:
    """Where the two consumers of an attention output leave the part of its gradient that is one ``[T, d]`` row per
    token, spread over the token's ``k`` slots with weight ``1/k``: ``grad`` from ``mid_source`` (the slot mean that
    feeds the next depth read), ``grad_running`` from ``layer_combine`` (the running mean). The attention backward
    adds both while it gathers rows, so neither is ever expanded to ``[T, k, d]``."""

    __slots__ = ("grad", "grad_running")

    def __init__(self) -> None:
        self.grad = None
        self.grad_running = None


class _Attention(torch.autograd.Function):
    """Packed varlen attention between the normed stream ``n [T, d]`` and gated slot updates."""

    # Head dims that are not multiples of 8 (30 at the 100m scale, 60 at 500m) break the 16-byte alignment TMA needs
    # for head starts and for the rows of W_o: such heads are re-pitched to the next multiple of 8 (zero-filled)
    # around the attention kernels, W_o is zero-padded along its inner dim for the GEMMs that read it, and its
    # gradient goes through a padded fp32 buffer.

    @staticmethod
    def forward(ctx, n, gates, wqkv, wo, tok_of_row, row_of_slot, slot_of_row_flat, pos_of_row, seg_start, col_start,
                groups, k, heads, head_dim, rope_base, mid_state=None):
        ctx.mid_state = mid_state
        T, d = n.shape
        inner = heads * head_dim
        hdp = -(-head_dim // 8) * 8
        pad = hdp != head_dim
        inner_p, inner8, n3 = heads * hdp, -(-inner // 8) * 8, -(-3 * inner // 8) * 8
        x = gather_rows(n, tok_of_row) if tok_of_row is not None else (n if n.dtype == BF16 else n.to(BF16))
        rows = x.shape[0]
        dev = x.device
        qkv = G.gemm_rows(x, wqkv, offsets=col_start, groups=groups, n=n3, out=G.rows_buffer(rows, n3, BF16, dev))
        rope_(qkv, pos_of_row, heads, head_dim, inner, rope_base, 1.0)
        att = repack_heads(qkv, 3 * heads, head_dim, hdp, 3 * inner_p) if pad else qkv
        q, kk, v = att[:, :inner_p], att[:, inner_p : 2 * inner_p], att[:, 2 * inner_p : 3 * inner_p]
        o_att, lse = flash.flash_fwd(q, kk, v, seg_start, heads, hdp, 1.0 / head_dim,
                                     out=G.rows_buffer(rows, inner_p, BF16, dev))
        o = repack_heads(o_att, heads, hdp, head_dim, inner8) if pad else o_att
        wo_use = torch.nn.functional.pad(wo, (0, inner8 - inner)) if inner8 != inner else wo
        y = G.gemm_rows(o, wo_use, offsets=col_start, groups=groups)
        gf = gates.float().contiguous().view(-1)
        out = combine_rows(y, row_of_slot.view(-1), gf, 1, T * k, round_products=False)
        ctx.save_for_backward(x, att, o_att, o, lse, y, gf, wqkv, wo_use, tok_of_row, row_of_slot, slot_of_row_flat,
                              pos_of_row, seg_start, col_start)
        ctx.meta = (groups, k, heads, head_dim, rope_base, T, n.dtype, gates.dtype)
        ctx.w_refs = (wqkv, wo)
        return out.view(T, k, d)

    @staticmethod
    def backward(ctx, dout):
        (x, att, o_att, o, lse, y, gf, wqkv, wo_use, tok_of_row, row_of_slot, slot_of_row_flat, pos_of_row, seg_start,
         col_start) = ctx.saved_tensors
        groups, k, heads, head_dim, rope_base, T, n_dtype, g_dtype = ctx.meta
        inner = heads * head_dim
        hdp = -(-head_dim // 8) * 8
        pad = hdp != head_dim
        inner_p, inner8, n3 = heads * hdp, -(-inner // 8) * 8, -(-3 * inner // 8) * 8
        d = y.shape[1]
        rows = x.shape[0]
        g2 = dout.contiguous().view(-1, d).float()
        # the gradient that reached this output through the slot mean (``mid_source``) was left in the shared state by
        # that node's backward; it is the same [T, d] row for the k slots of a token
        g_mid = g_run = None
        if ctx.mid_state is not None:
            g_mid, ctx.mid_state.grad = ctx.mid_state.grad, None
            g_run, ctx.mid_state.grad_running = ctx.mid_state.grad_running, None
        dy, dg_sorted = combine_bwd(g2, y, slot_of_row_flat, gf, 1, need_dw=ctx.needs_input_grad[1],
                                    shared=(g_mid, g_run), shared_div=k, shared_scale=1.0 / k)
        wq_ref, wo_ref = ctx.w_refs
        do = G.gemm_rows(dy, wo_use, offsets=col_start, groups=groups, b_mn=True, n=inner8,
                         out=G.rows_buffer(rows, inner8, BF16, dy.device))                     # wo [G, K=d, N=inner]
        d_wo = None
        if ctx.needs_input_grad[3]:
            if inner8 == inner:
                d_wo = _wgrad(dy, o, wo_ref, offsets=col_start, groups=groups)
            else:   # the gradient's rows would be misaligned for vector stores: reduce into a padded buffer first
                tmp = torch.empty(groups, d, inner8, dtype=torch.float32, device=dy.device)
                G.gemm_reduce(dy, o, offsets=col_start, groups=groups, out=tmp, epilogue=G.STORE_F32)
                part = tmp[..., :inner].reshape(wo_ref.shape)
                target = getattr(wo_ref, "_nb_grad", None)
                if target is not None:
                    target.add_(part)
                else:
                    d_wo = part.to(wo_ref.dtype)
        do_att = repack_heads(do, heads, head_dim, hdp, inner_p) if pad else do
        q, kk, v = att[:, :inner_p], att[:, inner_p : 2 * inner_p], att[:, 2 * inner_p : 3 * inner_p]
        dqkv = flash.flash_bwd(q, kk, v, o_att, do_att, lse, seg_start, heads, hdp, 1.0 / head_dim,
                               dqkv=G.rows_buffer(rows, 3 * inner_p, BF16, q.device))
        if pad:
            dqkv = repack_heads(dqkv, 3 * heads, hdp, head_dim, n3)
        rope_(dqkv, pos_of_row, heads, head_dim, inner, rope_base, -1.0)
        dq3 = dqkv[:, : 3 * inner]
        d_wqkv = _wgrad(dq3, x, wq_ref, offsets=col_start, groups=groups) if ctx.needs_input_grad[2] else None
        dn = None
        if ctx.needs_input_grad[0]:
            dx = G.gemm_rows(dq3, wqkv, offsets=col_start, groups=groups, b_mn=True, n=d)  # wqkv [G, K=3inner, N=d]
            if tok_of_row is not None:       # sum of the token's k packed rows, stored in the stream's dtype directly
                direct = n_dtype in (torch.float32, BF16)
                dn = combine_rows(dx, row_of_slot.view(-1), None, k, T, out_dtype=n_dtype if direct else torch.float32)
                dn = dn if direct else dn.to(n_dtype)
            else:
                dn = dx if dx.dtype == n_dtype else dx.to(n_dtype)
        dgates = None
        if dg_sorted is not None:
            dgates = dg_sorted.view(T, k).to(g_dtype)
        return (dn, dgates, d_wqkv, d_wo) + (None,) * 12


def column_attention(n, plan: ColumnPlan, gates, wqkv, wo, heads, head_dim, rope_base, cd, causal=True):
    if not causal:
        # the attention kernels mask above the diagonal of every segment; bidirectional attention runs the PyTorch statement
        _oracle_path("column_attention", "bidirectional (non-causal) attention")
        return ref.column_attention(n, plan, gates, wqkv, wo, heads, head_dim, rope_base, cd, causal=False)
    slot_flat = plan.extra.get("slot_flat")
    if slot_flat is None:   # flat (token*k + slot) index of every packed row
        slot_flat = (plan.tok_of_row * plan.k + plan.slot_of_row).contiguous()
        plan.extra["slot_flat"] = slot_flat
    state = _MidState() if torch.is_grad_enabled() else None
    out = _Attention.apply(n, gates, wqkv, wo, plan.tok_of_row, plan.row_of_slot, slot_flat, plan.pos_of_row,
                           plan.seg_start, plan.col_start, plan.G, plan.k, heads, head_dim, rope_base, state)
    if state is not None:
        out._nb_mid_state = state     # picked up by mid_source: its gradient for this tensor travels through the state
    return out


_dense_plans: dict = {}


def dense_attention(n, B, S, wqkv, wo, heads, head_dim, rope_base, cd, pos=None, causal=True):
    if not causal:
        _oracle_path("dense_attention", "bidirectional (non-causal) attention")
        return ref.dense_attention(n, B, S, wqkv, wo, heads, head_dim, rope_base, cd, pos=pos, causal=False)
    T = n.shape[0]
    key = (B, S, n.device)
    if key not in _dense_plans:
        ar = torch.arange(T, dtype=torch.int32, device=n.device)
        _dense_plans[key] = (ar, torch.arange(S, dtype=torch.int32, device=n.device).repeat(B),
                             torch.arange(0, T + 1, S, dtype=torch.int32, device=n.device),
                             torch.tensor([0, T], dtype=torch.int32, device=n.device))
    ar, p0, seg, col = _dense_plans[key]
    p = p0 if pos is None else pos.reshape(-1).clamp_min(0).to(torch.int32)
    ones = torch.ones(T, 1, dtype=torch.float32, device=n.device)
    out = _Attention.apply(n, ones, wqkv, wo, None, ar.view(T, 1), ar, p, seg, col, 1, 1, heads, head_dim, rope_base)
    return out.view(T, -1)


# ------------------------------------------------------------------------ LM head + CE
class _HeadCE(torch.autograd.Function):
    """Chunked head GEMM + cross-entropy; gradients are produced in the forward pass and scaled in backward."""

    @staticmethod
    def forward(ctx, hidden, weight, targets, multiplier: float, chunk_rows: int, ignore_index: int):
        T, d = hidden.shape
        V = weight.shape[0]
        ld = -(-V // 8) * 8
        bn = 256
        nt = -(-ld // bn)
        hb = hidden if hidden.dtype == BF16 else hidden.to(BF16)
        hb = hb.contiguous()
        dev = hidden.device
        need_grad = hidden.requires_grad or weight.requires_grad
        losses = torch.empty(T, dtype=torch.float32, device=dev)
        dh = torch.empty(T, d, dtype=BF16, device=dev) if need_grad else None
        dw = torch.empty(V, d, dtype=torch.float32, device=dev) if need_grad else None
        chunk = min(chunk_rows, T)
        logits = torch.empty(chunk, ld, dtype=BF16, device=dev)
        part = torch.empty(chunk, nt * G.STATS_PARTS, 2, dtype=torch.float32, device=dev)
        L = _L()
        for i, a in enumerate(range(0, T, chunk)):
            n = min(chunk, T - a)
            G.gemm_rows(hb[a : a + n], weight, out=logits[:n], epilogue=G.STORE_BF16_STATS, alpha=multiplier, bn=bn,
                        extra_out=(part,), n=ld, n_valid=V)
            _ck(L.nb_ce_grad(logits.data_ptr(), ld, V, part.data_ptr(), nt * G.STATS_PARTS, targets[a : a + n].data_ptr(), ignore_index,
                             losses[a : a + n].data_ptr(), n, _st()), "ce_grad")
            if need_grad:
                dl = logits[:n, :V] if ld == V else torch.as_strided(logits, (n, V), (ld, 1))
                G.gemm_rows(dl, weight, b_mn=True, out=dh[a : a + n], alpha=multiplier, n=d,
                            bn=_one_wave_bn(n, d))                                        # dH = dL . W
                G.gemm_reduce(dl, hb[a : a + n], out=dw, epilogue=G.STORE_F32 if i == 0 else G.ACCUM_F32,
                              alpha=multiplier)
        ctx.save_for_backward(dh, dw)
        ctx.h_dtype = hidden.dtype
        ctx.w_ref = weight
        count = (targets != ignore_index).sum()
        ctx.mark_non_differentiable(count)
        return losses.sum(), count

    @staticmethod
    def backward(ctx, g_loss, _g_count):
        dh, dw = ctx.saved_tensors
        d_hidden = (dh.float() * g_loss).to(ctx.h_dtype) if ctx.needs_input_grad[0] else None
        d_weight = None
        if ctx.needs_input_grad[1]:
            target = getattr(ctx.w_ref, "_nb_grad", None)
            if target is not None:
                target.addcmul_(dw, g_loss.to(dw.dtype).expand_as(dw))
            else:
                d_weight = (dw * g_loss).to(ctx.w_ref.dtype)
        return d_hidden, d_weight, None, None, None, None


def _one_wave_bn(rows: int, n: int, sms: int | None = None) -> int | None:
    """Widest 64-multiple tile width whose tile count still fits one wave of CTAs (long-K products)."""

    sms = _lib.sm_count() if sms is None else sms
    m_tiles = -(-rows // 128)
    best = None
    for bn in (64, 128, 192, 256):
        if m_tiles * -(-n // bn) <= sms:
            return bn if best is None else best
    return best


def lm_head_ce(hidden, weight, targets, multiplier, cd, chunk_rows=4096, ignore_index=-100):
    w = weight if weight.dtype == BF16 else weight.to(BF16)
    return _HeadCE.apply(hidden, w, targets.contiguous(), float(multiplier), int(chunk_rows), int(ignore_index))


# ------------------------------------------------------------------- depth read + norm
def _ptr_array(tensors):
    arr = (C.c_void_p * len(tensors))()
    for i, t in enumerate(tensors):
        arr[i] = t.data_ptr()
    return arr


class _SinkState:
    """Gradient buffer shared by every depth read of one source (see ``grad_sink``)."""

    __slots__ = ("buf",)

    def __init__(self) -> None:
        self.buf = None


class _GradSink(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, state):
        ctx.state = state
        ctx.set_materialize_grads(False)
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        st = ctx.state
        buf, st.buf = st.buf, None
        if buf is None:
            return g, None
        if g is not None:
            buf.add_(g)
        return buf, None


def grad_sink(x: Tensor) -> Tensor:
    """Mark ``x`` as a depth source read many times: the depth reads' backward passes add their
    gradients for it into one shared buffer (inside their kernel) instead of handing autograd one
    ``[T, d]`` tensor per read to sum. Autograd runs this node after every reader, where the
    buffer joins the gradient from ``x``'s other consumers."""

    if not (x.requires_grad and torch.is_grad_enabled() and x.dtype == torch.float32 and x.is_contiguous()):
        return x
    state = _SinkState()
    out = _GradSink.apply(x, state)
    out._nb_sink = state
    return out


KEEP_DEPTH_H = os.environ.get("NESTOR_DEPTH_READ_KEEP_H", "1") == "1"


class _DepthReadNorm(torch.autograd.Function):
    """One pass over the sources forward (online softmax over depth), three sweeps backward."""

    @staticmethod
    def forward(ctx, query, gains, gamma, eps_read, eps_norm, *sources):
        T, d = sources[0].shape
        n = len(sources)
        srcs = [s if (s.dtype == torch.float32 and s.is_contiguous()) else s.float().contiguous() for s in sources]
        out = torch.empty(T, d, dtype=BF16, device=srcs[0].device)
        stats = torch.empty(T, n, 2, dtype=torch.float32, device=out.device)
        rstd = torch.empty(T, dtype=torch.float32, device=out.device)
        q32, g32, w32 = query.float().contiguous(), gains.float().contiguous(), gamma.float().contiguous()
        # the mixture h is kept for the backward when anything needs a gradient (one [T, d] row per token instead of a
        # third pass over all n sources there); NESTOR_DEPTH_READ_KEEP_H=0 trades that memory back for the pass
        keep_h = KEEP_DEPTH_H and any(ctx.needs_input_grad)
        h = torch.empty(T, d, dtype=torch.float32, device=out.device) if keep_h else None
        _ck(_L().nb_depth_read_norm(_ptr_array(srcs), n, q32.data_ptr(), g32.data_ptr(), w32.data_ptr(), eps_read,
                                    eps_norm, out.data_ptr(), _ptr(h), stats.data_ptr(), rstd.data_ptr(), T, d, _st()),
            "depth_read_norm")
        ctx.kept_h = keep_h
        ctx.save_for_backward(q32, g32, w32, stats, rstd, *([h] if keep_h else []), *srcs)
        ctx.sinks = [getattr(s, "_nb_sink", None) if c is s else None for s, c in zip(sources, srcs)]
        ctx.dtypes = (query.dtype, gains.dtype, gamma.dtype, [s.dtype for s in sources])
        ctx.n_gains = gains.numel()
        return out

    @staticmethod
    def backward(ctx, dn):
        q32, g32, w32, stats, rstd, *srcs = ctx.saved_tensors
        h = srcs.pop(0) if ctx.kept_h else None
        n = len(srcs)
        T, d = srcs[0].shape
        # sources with a shared gradient buffer: the first reader to run backward creates it, later ones add
        outs, mask = [], 0
        for i, sink in enumerate(ctx.sinks):
            if sink is not None and ctx.needs_input_grad[5 + i]:
                if sink.buf is None:
                    sink.buf = torch.empty(T, d, dtype=torch.float32, device=dn.device)
                else:
                    mask |= 1 << i
                outs.append(sink.buf)
            else:
                outs.append(torch.empty(T, d, dtype=torch.float32, device=dn.device))
        dq = torch.empty(d, dtype=torch.float32, device=dn.device)
        dg = torch.zeros(ctx.n_gains, dtype=torch.float32, device=dn.device)     # gains past the n sources read get no gradient
        dw = torch.empty(d, dtype=torch.float32, device=dn.device)
        scratch = torch.empty(8 * _lib.sm_count(dn.device) * (2 * d + 64), dtype=torch.float32, device=dn.device)
        dnb = dn if (dn.dtype == BF16 and dn.is_contiguous()) else dn.to(BF16).contiguous()
        _ck(_L().nb_depth_read_norm_bwd(_ptr_array(srcs), _ptr_array(outs), n, q32.data_ptr(),
                                        g32.data_ptr(), w32.data_ptr(), stats.data_ptr(), rstd.data_ptr(), dnb.data_ptr(),
                                        None, dq.data_ptr(), dg.data_ptr(), dw.data_ptr(), T, d, C.c_ulonglong(mask),
                                        scratch.data_ptr(), _ptr(h), _st()),
            "depth_read_norm_bwd")
        _lib.count_launch()
        qd, gd, wd, sd = ctx.dtypes
        grads = [None if (sink is not None and ctx.needs_input_grad[5 + i]) else g.to(t)
                 for i, (g, t, sink) in enumerate(zip(outs, sd, ctx.sinks))]
        return (dq.to(qd), dg.to(gd), dw.to(wd), None, None, *grads)


def depth_read_norm(sources, query, gains, gamma, eps_read, eps_norm, out_dtype, key_cache=None):
    # (a key cache is accepted and ignored: the kernel derives every source's scale inside its one pass)
    if out_dtype != BF16:
        raise RuntimeError("the fused depth-read kernel writes bf16; run full-precision evaluation under ops.oracle_ops()")
    if query.dim() == 2:
        # one query row per source: the fused kernel scores every source with one shared vector
        _oracle_path("depth_read_norm", "per-source queries")
        return ref.depth_read_norm(sources, query, gains, gamma, eps_read, eps_norm, out_dtype)
    return _DepthReadNorm.apply(query, gains, gamma, float(eps_read), float(eps_norm), *sources)


# --------------------------------------------------------------------- stream updates
def _f32c(t):
    return t if (t.dtype == torch.float32 and t.is_contiguous()) else t.float().contiguous()


class _MidSource(torch.autograd.Function):
    """``running + mean_j attn_j``. The attention output has a second consumer (``layer_combine``), so autograd would
    add this node's broadcast gradient ``g / k`` to the other one with a pass over ``[T, k, d]``. When the attention
    op offers a shared state, the ``[T, d]`` gradient is parked there instead and the attention backward, which
    autograd runs after both consumers, adds it while it gathers its rows."""

    @staticmethod
    def forward(ctx, running, attn, state=None):
        ctx.state = state
        T, k, d = attn.shape
        a = _f32c(attn)
        r = None if running is None else _f32c(running)
        out = torch.empty(T, d, dtype=torch.float32, device=attn.device)
        _ck(_L().nb_mid_source(_ptr(r), a.data_ptr(), out.data_ptr(), T, d, k, _st()), "mid_source")
        ctx.k = k
        ctx.has_running = running is not None
        return out

    @staticmethod
    def backward(ctx, g):
        k = ctx.k
        d_run = g if ctx.has_running and ctx.needs_input_grad[0] else None
        if ctx.state is not None:
            ctx.state.grad = g if g.is_contiguous() else g.contiguous()
            return d_run, None, None
        return d_run, (g * (1.0 / k)).unsqueeze(1).expand(-1, k, -1), None


def mid_source(running, attn):
    return _MidSource.apply(running, attn, getattr(attn, "_nb_mid_state", None))


class _LayerCombine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, attn, priv, pub, path, streams, running, attn_state=None):
        ctx.attn_state = attn_state
        T, k, d = attn.shape
        a, pb = _f32c(attn), _f32c(pub)
        pv = None if priv is None else _f32c(priv)
        ph = None if path is None else _f32c(path)
        st = None if streams is None else _f32c(streams)
        rn = None if running is None else _f32c(running)
        s_out = torch.empty(T, k, d, dtype=torch.float32, device=attn.device)
        r_out = torch.empty(T, d, dtype=torch.float32, device=attn.device)
        _ck(_L().nb_layer_combine(a.data_ptr(), _ptr(pv), pb.data_ptr(), _ptr(ph), _ptr(st), _ptr(rn), s_out.data_ptr(),
                                  r_out.data_ptr(), T, d, k, _st()), "layer_combine")
        ctx.save_for_backward(pv, pb, ph)
        ctx.shape = (T, k, d)
        ctx.has_state = (streams is not None, running is not None)
        return s_out, r_out

    @staticmethod
    def backward(ctx, ds, dr):
        pv, pb, ph = ctx.saved_tensors
        T, k, d = ctx.shape
        dev = pb.device
        ds_c = None if ds is None else _f32c(ds)
        dr_c = None if dr is None else _f32c(dr)
        # d_attn = ds + dr / k. When the attention op offers its shared state, ds itself is handed on as the gradient
        # and dr is parked for the attention backward to add, which saves writing (and re-reading) a [T, k, d] tensor
        park = ctx.attn_state is not None and ds_c is not None
        d_attn = None if park else torch.empty(T, k, d, dtype=torch.float32, device=dev)
        d_priv = torch.empty(T, k, d, dtype=torch.float32, device=dev) if pv is not None else None
        d_pub = torch.empty(T, d, dtype=torch.float32, device=dev)
        d_path = torch.empty(T, 2, dtype=torch.float32, device=dev) if ph is not None else None
        _ck(_L().nb_layer_combine_bwd(_ptr(ds_c), _ptr(dr_c), _ptr(pv), pb.data_ptr(), _ptr(ph), _ptr(d_attn),
                                      _ptr(d_priv), d_pub.data_ptr(), _ptr(d_path), T, d, k, _st()), "layer_combine_bwd")
        if park:
            ctx.attn_state.grad_running = dr_c
            d_attn = ds_c
        return (d_attn, d_priv, d_pub, d_path, ds if ctx.has_state[0] else None, dr if ctx.has_state[1] else None, None)


def layer_combine(attn, priv, pub, path, streams, running, cd):
    return _LayerCombine.apply(attn, priv, pub, path, streams, running, getattr(attn, "_nb_mid_state", None))


class _BlockExit(torch.autograd.Function):
    @staticmethod
    def forward(ctx, streams):
        T, k, d = streams.shape
        s = _f32c(streams)
        dev_ = torch.empty(k, T, d, dtype=torch.float32, device=s.device)
        agg = torch.empty(T, d, dtype=torch.float32, device=s.device)
        _ck(_L().nb_block_exit(s.data_ptr(), dev_.data_ptr(), agg.data_ptr(), T, d, k, _st()), "block_exit")
        ctx.shape = (T, k, d)
        return dev_, agg

    @staticmethod
    def backward(ctx, d_dev, d_agg):
        T, k, d = ctx.shape
        dd = None if d_dev is None else _f32c(d_dev)
        da = None if d_agg is None else _f32c(d_agg)
        out = torch.empty(T, k, d, dtype=torch.float32, device=(dd if dd is not None else da).device)
        _ck(_L().nb_block_exit_bwd(_ptr(dd), _ptr(da), out.data_ptr(), T, d, k, _st()), "block_exit_bwd")
        return out


def block_exit(streams):
    return _BlockExit.apply(streams)


# ------------------------------------------------------------------------------ plans
def build_column_plan(idx, G_, pos=None):
    """Packed-attention plan by a counting sort on (column, sequence) keys: five small kernels."""

    B, S, k = idx.shape
    if G_ * B > 256:
        _oracle_path("build_column_plan", f"columns x sequences = {G_ * B} exceeds the 256 sort keys of the counting-sort kernels")
        return ref.build_column_plan(idx, G_, pos)
    dev = idx.device
    T, n = B * S, B * S * k
    i32 = torch.int32
    idx32 = idx.reshape(T, k).to(i32).contiguous()
    p32 = None if pos is None else pos.reshape(-1).to(i32).contiguous()
    keys, order, inv = (torch.empty(n, dtype=i32, device=dev) for _ in range(3))
    tok, slot, prow = (torch.empty(n, dtype=i32, device=dev) for _ in range(3))
    seg = torch.empty(G_ * B + 1, dtype=i32, device=dev)
    scratch = torch.empty(max(1, -(-n // 1024)) * G_ * B, dtype=i32, device=dev)
    _ck(_L().nb_column_plan(idx32.data_ptr(), T, k, S, B, G_, _ptr(p32), keys.data_ptr(), scratch.data_ptr(),
                            order.data_ptr(), inv.data_ptr(), seg.data_ptr(), tok.data_ptr(), slot.data_ptr(),
                            prow.data_ptr(), _st()), "column_plan")
    _lib.count_launch(4)
    return ColumnPlan(B=B, S=S, G=G_, k=k, idx=idx32, row_of_slot=inv.view(T, k), tok_of_row=tok, slot_of_row=slot,
                      pos_of_row=prow, seg_start=seg, col_start=seg[::B].contiguous(),
                      extra={"slot_flat": order})      # the sorted flat (token * k + slot) index of every packed row


def build_expert_plan(expert_ids, E):
    """Counting sort by expert (three small kernels; the oracle sorts)."""

    if E > 256:
        _oracle_path("build_expert_plan", f"{E} experts exceed the 256 sort keys of the counting-sort kernels")
        return ref.build_expert_plan(expert_ids, E)
    T, slots = expert_ids.shape
    ids = expert_ids.reshape(-1)
    if ids.dtype != torch.int32:
        ids = ids.to(torch.int32)
    ids = ids.contiguous()
    n = ids.numel()
    dev = ids.device
    order = torch.empty(n, dtype=torch.int32, device=dev)
    inv = torch.empty(n, dtype=torch.int32, device=dev)
    offsets = torch.empty(E + 1, dtype=torch.int32, device=dev)
    scratch = torch.empty(max(1, -(-n // 1024)) * E, dtype=torch.int32, device=dev)
    L = _L()
    _ck(L.nb_expert_plan(ids.data_ptr(), n, E, scratch.data_ptr(), order.data_ptr(), inv.data_ptr(), offsets.data_ptr(),
                         _st()), "expert_plan")
    _lib.count_launch(2)
    return ExpertPlan(E=E, n=n, slots=slots, order=order, inv=inv, offsets=offsets)


# ---------------------------------------------------------------------------- routing
class RouteArgs(C.Structure):
    _fields_ = [("scores", C.c_void_p), ("ld", C.c_long), ("is_f32", C.c_int), ("col_off", C.c_int),
                ("cols", C.c_void_p), ("k_cols", C.c_int), ("bias", C.c_void_p),
                ("E", C.c_int), ("k", C.c_int), ("mode", C.c_int), ("T", C.c_int),
                ("idx_in", C.c_void_p), ("idx_out", C.c_void_p), ("id_out", C.c_void_p), ("gates", C.c_void_p),
                ("colgate", C.c_void_p), ("w_out", C.c_void_p)]


_MODES = {"renorm": 0, "switch": 1, "all": 2}


def _route_args(scores, E, k, mode, cols, bias, idx_in, idx, ids, gates, colgate, w) -> RouteArgs:
    a = RouteArgs()
    a.scores, a.ld, a.is_f32, a.col_off = scores.data_ptr(), scores.stride(0), int(scores.dtype == torch.float32), 0
    a.cols, a.k_cols = _ptr(cols), (cols.shape[1] if cols is not None else 1)
    a.bias = _ptr(bias)
    a.E, a.k, a.mode, a.T = E, k, mode, scores.shape[0]
    a.idx_in, a.idx_out, a.id_out, a.gates = _ptr(idx_in), idx.data_ptr(), _ptr(ids), gates.data_ptr()
    a.colgate, a.w_out = _ptr(colgate), _ptr(w)
    return a


class _Route(torch.autograd.Function):
    """Top-k selection + gates of one router family in one kernel (and one for the backward)."""

    @staticmethod
    def forward(ctx, scores, bias, cols, colgate, k: int, mode: int, idx_in, want_w: bool):
        # scores: [T, E] (stride(1) == 1, any row pitch) or, with a column selection, [T, G, E] (E contiguous, G*E per row)
        sel = cols is not None
        E = scores.shape[-1]
        T = scores.shape[0]
        assert scores.stride(-1) == 1 and scores.dtype in (BF16, torch.float32)
        if sel:
            assert scores.ndim == 3 and scores.stride(1) == E
            cols = cols.to(torch.int32).contiguous()
            colgate = colgate.float().contiguous()
        nprob = T * (cols.shape[1] if sel else 1)
        dev = scores.device
        idx = torch.empty(nprob, k, dtype=torch.int32, device=dev)
        gates = torch.empty(nprob, k, dtype=torch.float32, device=dev)
        ids = torch.empty(nprob, k, dtype=torch.int32, device=dev) if sel else None
        w = torch.empty(nprob, k, dtype=BF16, device=dev) if want_w else None
        b = bias.float().contiguous() if bias is not None else None
        ii = idx_in.to(torch.int32).contiguous() if idx_in is not None else None
        a = _route_args(scores, E, k, mode, cols if sel else None, b, ii, idx, ids, gates, colgate if sel else None, w)
        _ck(_L().nb_route_fwd(C.byref(a), _st()), "route_fwd")
        ctx.save_for_backward(scores, idx, gates, cols if sel else None, colgate if sel else None, b)
        ctx.meta = (E, k, mode, sel, want_w)
        ctx.mark_non_differentiable(idx)
        if ids is not None:
            ctx.mark_non_differentiable(ids)
        return idx, gates, ids, w

    @staticmethod
    def backward(ctx, _d_idx, d_gates, _d_ids, d_w):
        scores, idx, gates, cols, colgate, b = ctx.saved_tensors
        E, k, mode, sel, want_w = ctx.meta
        dscores = torch.zeros(scores.shape, dtype=scores.dtype, device=scores.device)
        dcolgate = torch.empty(colgate.shape, dtype=torch.float32, device=scores.device) if sel else None
        a = _route_args(scores, E, k, mode, cols, b, None, idx, None, gates, colgate, None)
        dg = d_gates.float().contiguous() if d_gates is not None else None
        dw = d_w.contiguous() if d_w is not None else None
        # the gradient buffer is dense over this family's columns: its own row pitch, same block layout
        ld_d = dscores.stride(0)
        a_d = RouteArgs.from_buffer_copy(a)
        _ck(_L().nb_route_bwd(C.byref(a_d), _ptr(dg), _ptr(dw), dscores.data_ptr(), ld_d,
                              int(dscores.dtype == torch.float32), _ptr(dcolgate), _st()), "route_bwd")
        return dscores, None, None, dcolgate, None, None, None, None


def route_topk(scores: Tensor, bias: Tensor, k: int, gate_mode: str):
    """Kernel body of ``reference.route_topk`` for 2-D score matrices (others take the oracle path)."""

    if scores.ndim != 2 or scores.shape[-1] > 64 or k > 8 or scores.stride(-1) != 1:
        _oracle_path("route_topk", f"scores {tuple(scores.shape)} stride {scores.stride()} k={k}: the routing kernel takes 2-D "
                                   "row-major scores with at most 64 candidates and k <= 8")
        return ref.route_topk(scores, bias, k, gate_mode)
    tape = ref._TAPE
    idx_in = None
    if tape is not None and tape.mode == "replay":
        idx_in = tape.selections[tape.cursor]
        tape.cursor += 1
    idx, gates, _, _ = _Route.apply(scores, bias, None, None, k, _MODES[gate_mode], idx_in, False)
    if tape is not None and tape.mode == "record":
        tape.selections.append(idx.long())
    return idx, gates


def route_selected(scores: Tensor, bias: Tensor, cols: Tensor, col_gates: Tensor, k: int, gate_mode: str, cd):
    T, Gn, Q = scores.shape
    if Q > 64 or k > 8 or scores.stride(-1) != 1 or scores.stride(1) != Q or cd != BF16:
        _oracle_path("route_selected", f"scores {tuple(scores.shape)} k={k} dtype {cd}: the routing kernel takes packed bf16-path "
                                       "scores with at most 64 experts per column and k <= 8")
        return ref.route_selected(scores, bias, cols, col_gates, k, gate_mode, cd)
    kc = cols.shape[1]
    tape = ref._TAPE
    idx_in = None
    if tape is not None and tape.mode == "replay":
        idx_in = tape.selections[tape.cursor].reshape(T * kc, k)
        tape.cursor += 1
    idx, _gates, ids, w = _Route.apply(scores, bias, cols, col_gates, k, _MODES[gate_mode], idx_in, True)
    if tape is not None and tape.mode == "record":
        tape.selections.append(idx.long().view(T, kc, k))
    return ids.view(T, kc * k), w.view(T, kc * k), idx.view(T, kc, k)


# ---------------------------------------------------------------------- Newton-Schulz
_NS_MAX_BATCH = 256      # groups per grouped-GEMM launch


@torch.no_grad()
def newton_schulz(g: Tensor, steps: int = 5, out_dtype: torch.dtype | None = None) -> Tensor:
    """Quintic Newton-Schulz on ``[..., m, n]`` matrices, every product on the tcgen05 grouped GEMM.

    One batch (up to 256 same-shape matrices) costs ``3 + 3 * steps`` launches: normalise + cast + orient
    (``nb_ns_prepare``), then per iteration ``A = X X^T`` (K-major B = X), ``B = b A + c A A`` and
    ``X <- a X + B X`` (B operand X read MN-major), the last two through the ``alpha * acc + beta * E1``
    epilogue, then ``nb_ns_finish`` when the result has to be turned back or un-padded. Matrices are the
    groups of the launches; rows of a matrix shorter than a 128-row tile are masked, not padded.
    """

    a, b, c = ref.NS_COEFFS
    squeeze = g.ndim == 2
    x = g.unsqueeze(0) if squeeze else g
    if x.ndim != 3:
        x = x.reshape(-1, *x.shape[-2:])
    x = x.float().contiguous()
    Bt, m, n = x.shape
    rows, cols = min(m, n), max(m, n)
    mp, npad = -(-rows // 8) * 8, -(-cols // 8) * 8
    direct = m <= n and mp == m and npad == n      # the iterate already has the parameter's layout
    dev = x.device
    out = torch.empty(Bt, m, n, dtype=BF16, device=dev)
    L = _L()
    for lo in range(0, Bt, _NS_MAX_BATCH):
        nb = min(_NS_MAX_BATCH, Bt - lo)
        X = out[lo : lo + nb].view(nb * mp, npad) if direct and steps % 2 == 0 else torch.empty(nb * mp, npad, dtype=BF16, device=dev)
        X2 = out[lo : lo + nb].view(nb * mp, npad) if direct and steps % 2 == 1 else torch.empty(nb * mp, npad, dtype=BF16, device=dev)
        A = torch.empty(nb * mp, mp, dtype=BF16, device=dev)
        Bm = torch.empty(nb * mp, mp, dtype=BF16, device=dev)
        partial = torch.empty(nb * 32, dtype=torch.float32, device=dev)
        _ck(L.nb_ns_prepare(x[lo : lo + nb].data_ptr(), X.data_ptr(), nb, m, n, mp, npad, partial.data_ptr(), _st()), "ns_prepare")
        for _ in range(steps):
            G.gemm_rows(X, X.view(nb, mp, npad), groups=nb, out=A)
            G.gemm_rows(A, A.view(nb, mp, mp), groups=nb, out=Bm, epilogue=G.AXPBY_BF16, alpha=c, beta=b, extra_in=(A,))
            G.gemm_rows(Bm, X.view(nb, mp, npad), groups=nb, b_mn=True, n=npad, out=X2, epilogue=G.AXPBY_BF16,
                        alpha=1.0, beta=a, extra_in=(X,))
            X, X2 = X2, X
        if not direct:
            _ck(L.nb_ns_finish(X.data_ptr(), out[lo : lo + nb].data_ptr(), nb, m, n, mp, npad, _st()), "ns_finish")
    out = out.view(g.shape)
    want = g.dtype if out_dtype is None else out_dtype
    return out if want == BF16 else out.to(want)
