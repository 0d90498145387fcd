"""Micro-benchmarks of the sm_100a kernels on the model's own shapes (CUDA events, warm-up, L2-sized inputs).

``python -m nestor_b200.scripts.bench_kernels [case ...] [--reps N]`` prints one line per kernel launch
shape: time, achieved TFLOP/s or GB/s and the fraction of the measured peaks in ``MEASURED_PEAKS.json``
(fallback 1590 TFLOP/s, 6650 GB/s). Cases: ``gemm`` (expert / attention / head GEMMs of nestor_200m),
``flash``, ``depth``, ``ns`` (Newton-Schulz), ``gather`` (all-gather fused into the bank GEMMs, one GPU), ``small`` /
``gather-small`` (one launch of each, sized for a profiler capture). Inputs are larger
than the 126 MB L2 or an L2 flush is written between repetitions.
"""

from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch

BF = torch.bfloat16


def peaks() -> tuple[float, float, str]:
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.is_file():
        d = json.loads(p.read_text())
        return float(d["bf16_tflops"]), float(d["hbm_gbs"]), "measured"
    return 1590.0, 6650.0, "fallback"


_flush = None
WARMUP = 3


def timed(fn, reps: int, flush: bool = True) -> float:
    """Mean device time of ``fn`` in ms. Every repetition (L2 flush, start event, ``fn``, stop event) is enqueued behind
    a spin kernel before anything is waited for, so the host is always ahead of the device: the events bracket the
    kernels of ``fn`` and nothing else. (With a synchronise per repetition the start event completes on an idle GPU
    and the host time of the Python launch path, some 50 us, is counted as kernel time.)"""

    global _flush
    if flush and _flush is None:
        _flush = torch.empty(160 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    for _ in range(WARMUP):
        fn()
    torch.cuda.synchronize()
    pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
    torch.cuda._sleep(4_000_000)          # about 2 ms of device time for the host to get ahead
    for e0, e1 in pairs:
        if flush:
            _flush.zero_()
        e0.record(); fn(); e1.record()
    torch.cuda.synchronize()
    return sum(e0.elapsed_time(e1) for e0, e1 in pairs) / reps


def offsets(rows: int, groups: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(0)
    c = torch.full((groups,), rows // groups, dtype=torch.int64)
    j = ((torch.rand(groups, generator=g) * 0.3 - 0.15) * (rows // groups)).long()
    c = (c + j - j.sum() // groups).clamp_min(0)
    c[-1] += rows - c.sum()
    o = torch.zeros(groups + 1, dtype=torch.int32)
    o[1:] = c.cumsum(0)
    return o.cuda()


def report(name: str, ms: float, flops: float = 0.0, nbytes: float = 0.0) -> None:
    tf, gb, src = peaks()
    parts = [f"{name:58s} {ms * 1e3:9.1f} us"]
    if flops:
        parts.append(f"{flops / ms / 1e9:7.0f} TF/s ({flops / ms / 1e9 / tf:5.1%} of {src} bf16 peak)")
    if nbytes:
        parts.append(f"{nbytes / ms / 1e6:7.0f} GB/s ({nbytes / ms / 1e6 / gb:5.1%} of {src} HBM)")
    print("  ".join(parts), flush=True)


def case_gemm(reps: int, small: bool = False) -> None:
    from nestor_b200.ops import gemm as G
    T, d = (4096 if small else 16384), 640
    for k, kq, h, H in ([(3, 2, 216, 5)] if small else [(3, 2, 216, 5), (6, 1, 216, 3), (8, 1, 160, 2)]):
        E, n = 64, T * k * kq
        off = offsets(n, E)
        X = torch.randn(n, d, device="cuda").to(BF)
        Wg, Wu = torch.randn(E, d, h, device="cuda").to(BF), torch.randn(E, d, h, device="cuda").to(BF)
        Wd = torch.randn(E, h, d, device="cuda").to(BF)
        Hh = torch.empty(n, h, device="cuda", dtype=BF)
        Gt, Ut, Y = torch.empty_like(Hh), torch.empty_like(Hh), torch.empty(n, d, device="cuda", dtype=BF)
        report(f"private k={k} up|gate+SwiGLU [{n}x{d}]x[{E},{d},{2 * h}]", timed(lambda: G.gemm_rows(
            X, Wg, B2=Wu, offsets=off, groups=E, b_mn=True, out=Hh, epilogue=G.SWIGLU, extra_out=(Gt, Ut)), reps), 4.0 * n * d * h)
        report(f"private k={k} down [{n}x{h}]x[{E},{h},{d}]", timed(lambda: G.gemm_rows(
            Hh, Wd, offsets=off, groups=E, b_mn=True, out=Y), reps), 2.0 * n * d * h)
        gw = torch.zeros(E, d, h, device="cuda")
        report(f"private k={k} weight grad [{d}x{h}] x{E}", timed(lambda: G.gemm_reduce(X, Gt, offsets=off, groups=E, out=gw), reps),
               2.0 * n * d * h)
        inner, rows, Gc = H * 40, T * k, 8
        offc = offsets(rows, Gc)
        Xa = torch.randn(rows, d, device="cuda").to(BF)
        Wqkv, Wo = torch.randn(Gc, 3 * inner, d, device="cuda").to(BF), torch.randn(Gc, d, inner, device="cuda").to(BF)
        qkv = torch.empty(rows, 3 * inner, device="cuda", dtype=BF)
        o, y = torch.randn(rows, inner, device="cuda").to(BF), torch.empty(rows, d, device="cuda", dtype=BF)
        report(f"attention k={k} qkv [{rows}x{d}]x[8,{3 * inner},{d}]", timed(lambda: G.gemm_rows(
            Xa, Wqkv, offsets=offc, groups=Gc, out=qkv), reps), 6.0 * rows * d * inner)
        report(f"attention k={k} out [{rows}x{inner}]x[8,{d},{inner}]", timed(lambda: G.gemm_rows(
            o, Wo, offsets=offc, groups=Gc, out=y), reps), 2.0 * rows * d * inner)
    if small:
        return
    V, ld, ch = 100263, 100264, 4096
    Hd, W = torch.randn(ch, d, device="cuda").to(BF), torch.randn(V, d, device="cuda").to(BF)
    lg, part = torch.empty(ch, ld, device="cuda", dtype=BF), torch.empty(ch, 392 * G.STATS_PARTS, 2, device="cuda")
    report("head logits + softmax statistics [4096x640]x[100263,640]", timed(lambda: G.gemm_rows(
        Hd, W, out=lg, epilogue=G.STORE_BF16_STATS, alpha=0.125, bn=256, extra_out=(part,), n=ld, n_valid=V), reps), 2.0 * ch * d * V)
    A, B = torch.randn(8192, 8192, device="cuda").to(BF), torch.randn(8192, 8192, device="cuda").to(BF)
    out = torch.empty(8192, 8192, device="cuda", dtype=BF)
    report("square 8192^3", timed(lambda: G.gemm_rows(A, B, out=out), reps), 2.0 * 8192 ** 3)


def case_flash(reps: int, small: bool = False) -> None:
    from nestor_b200.ops import flash as F
    for H, hd, L, nseg in ([(5, 40, 1536, 8)] if small else [(5, 40, 1536, 32), (3, 40, 3072, 32), (2, 40, 4096, 32)]):
        rows, inner = L * nseg, H * hd
        qkv = torch.randn(rows, 3 * inner, device="cuda").to(BF)
        seg = torch.arange(0, rows + 1, L, dtype=torch.int32, device="cuda")
        q, k, v = qkv[:, :inner], qkv[:, inner:2 * inner], qkv[:, 2 * inner:]
        fl = nseg * H * 2.0 * L * L * hd          # causal: half of 2 * 2 * L^2 * hd
        report(f"flash forward H={H} hd={hd} {nseg}x{L}", timed(lambda: F.flash_fwd(q, k, v, seg, H, hd, 1 / hd), reps), fl)
        o, lse = F.flash_fwd(q, k, v, seg, H, hd, 1 / hd)
        do = torch.randn_like(o)
        report(f"flash backward H={H} hd={hd} {nseg}x{L}", timed(lambda: F.flash_bwd(q, k, v, o, do, lse, seg, H, hd, 1 / hd), reps), 2.5 * fl)


def case_depth(reps: int, small: bool = False) -> None:
    from nestor_b200.ops import cuda as K
    T, d = (4096 if small else 16384), 640
    for n in ([5] if small else [3, 8, 47]):
        srcs = [torch.randn(T, d, device="cuda", requires_grad=True) for _ in range(n)]
        q, gn, gm = (torch.randn(d, device="cuda") * 0.1).requires_grad_(), torch.ones(47, device="cuda", requires_grad=True), \
            torch.ones(d, device="cuda", requires_grad=True)
        report(f"depth read + norm forward, {n} sources [{T}x{d}]", timed(
            lambda: K.depth_read_norm([s.detach() for s in srcs], q.detach(), gn.detach(), gm.detach(), 1e-6, 1e-5, BF), reps),
            nbytes=(n * 4 + 2) * T * d)
        out = K.depth_read_norm(srcs, q, gn, gm, 1e-6, 1e-5, BF)
        g = torch.randn_like(out)
        report(f"depth read + norm backward, {n} sources", timed(lambda: torch.autograd.grad(out, srcs, g, retain_graph=True), reps),
               nbytes=(n * 8 + 2) * T * d)


def case_ns(reps: int, small: bool = False) -> None:
    """Newton-Schulz (5 iterations) on the Muon shape buckets of nestor_200m: the tcgen05 grouped-GEMM path against
    the same iteration on ``torch.bmm`` (the PyTorch statement of the op)."""

    from nestor_b200.ops import cuda as K, reference as R
    shapes = [(8, 200, 640)] if small else [(96, 200, 640), (96, 640, 200), (408, 640, 640), (512, 640, 216), (512, 216, 640), (7, 128, 640)]
    for bt, m, n in shapes:
        g = torch.randn(bt, m, n, device="cuda")
        r, c = min(m, n), max(m, n)
        fl = 5.0 * bt * (4.0 * r * r * c + 2.0 * r ** 3)
        report(f"newton-schulz x5 tcgen05 [{bt},{m},{n}]", timed(lambda: K.newton_schulz(g, 5, out_dtype=BF), reps, flush=False), fl)
        report(f"newton-schulz x5 torch.bmm [{bt},{m},{n}]", timed(lambda: R.newton_schulz(g, 5, out_dtype=BF), reps, flush=False), fl)


def case_gather(reps: int, small: bool = False) -> None:
    """Cost of the staging mechanism of the fused all-gather GEMM by itself: every "rank" is this GPU.

    The expert-bank products of nestor_200m, once reading their weights in place and once with the weights staged
    through the copy warps of the same launch (``ops.gemm.Gather`` whose eight sources all point at the local
    arena), so that no byte crosses NVLink and the difference is the price of the in-kernel copy and hand-off.
    """

    from nestor_b200.ops import gemm as G
    E, d, h, rows = 64, 640, 216, (24576 if small else 98304)
    n = E * d * h
    arena = (torch.randn(3 * n, device="cuda") * 0.03).to(BF)
    vg, vu, vd = arena[:n].view(E, d, h), arena[n : 2 * n].view(E, d, h), arena[2 * n :].view(E, h, d)
    X, Hh = torch.randn(rows, d, device="cuda").to(BF), torch.randn(rows, h, device="cuda").to(BF)
    off = (torch.arange(E + 1, dtype=torch.int32) * (rows // E)).cuda()
    H, Gt, Ut = (G.rows_buffer(rows, h, BF, "cuda") for _ in range(3))
    Y = torch.empty(rows, d, dtype=BF, device="cuda")
    stage = torch.empty(2 * n, dtype=BF, device="cuda")
    flags = torch.zeros(257, dtype=torch.int32, device="cuda")

    def up(g):
        G.gemm_rows(X, vg, B2=vu, offsets=off, groups=E, b_mn=True, out=H, epilogue=G.SWIGLU, extra_out=(Gt, Ut), gather=g)

    def down(g):
        G.gemm_rows(Hh, vd, offsets=off, groups=E, b_mn=True, out=Y, gather=g)

    report("up|gate+SwiGLU, weights in place", timed(lambda: up(None), reps), 2.0 * rows * d * 2 * h)
    report("down, weights in place", timed(lambda: down(None), reps), 2.0 * rows * d * h)
    for chunk, nbuf, lanes in ((8192, 4, 1), (32768, 2, 1), (8192, 2, 4)):
        spec = G.Gather(src=[arena.data_ptr()] * 8, arena_ptr=arena.data_ptr(), stage=stage, flags=flags,
                        groups_per_rank=E // 8, chunk=chunk, nbuf=nbuf, lanes=lanes)
        ring = f"{chunk} B x {nbuf} x {lanes} lane(s)"
        report(f"up|gate+SwiGLU, weights staged (ring {ring})", timed(lambda: up(spec), reps), 2.0 * rows * d * 2 * h)
        report(f"down, weights staged (ring {ring})", timed(lambda: down(spec), reps), 2.0 * rows * d * h)


def main(argv: list[str] | None = None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("cases", nargs="*", default=["gemm", "flash", "depth"])
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3, help="untimed launches per shape (0 under a profiler: one launch per shape)")
    a = ap.parse_args(argv)
    global WARMUP
    WARMUP = a.warmup
    torch.manual_seed(0)
    for c in a.cases:
        if c == "small":
            case_gemm(a.reps, small=True); case_flash(a.reps, small=True); case_depth(a.reps, small=True); case_ns(a.reps, small=True)
        else:
            {"gemm": case_gemm, "flash": case_flash, "depth": case_depth, "gather": case_gather, "ns": case_ns,
             "gather-small": lambda r: case_gather(r, small=True)}[c](a.reps)
    from nestor_b200.ops import _lib
    _lib.check_status(torch.device("cuda"))


if __name__ == "__main__":
    main()
