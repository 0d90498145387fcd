"""Micro-benchmark of the in-kernel collectives against NCCL (gradient all-reduce + cast, parameter push).

``torchrun --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 -m nestor_b200.scripts.bench_collectives``
(or ``python -m nestor_b200.scripts.bench_collectives`` for the one-rank local leg of each kernel) times, for 1 MB ... 1 GB fp32 buffers: the all-reduce kernel (fp32 sum, 1/W scale, optional bf16 mirror) and
``torch.distributed.all_reduce`` (NCCL) on the same buffer, the reduce-scatter onto per-rank ranges against
``reduce_scatter_tensor``, and the parameter push (all-gather fused with the bf16 cast) against
``all_gather_into_tensor`` + cast. Each of ours is timed on plain peer loads/stores and, when the symmetric buffers
have an NVLink multicast mapping, on ``multimem`` instructions. Device-timed with CUDA events, max over ranks.
Bus bandwidth is ``2 (W-1)/W * bytes / time`` for the all-reduce and ``(W-1)/W * bytes / time`` for the
gather; the roofline is the measured peer copy of 770 GB/s per direction per GPU (900 nominal).
"""

from __future__ import annotations

import argparse
import os

import torch
import torch.distributed as dist

PEER_COPY_GBS = 770.0


def timed(fn, reps: int, dev, per_rank: list | None = None) -> float:
    for _ in range(3):
        fn()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / reps], device=dev)
    if per_rank is not None:          # every rank's own time, for launches whose cost depends on the rank
        every = [torch.zeros_like(t) for _ in range(dist.get_world_size())]
        dist.all_gather(every, t)
        per_rank.extend(float(x.item()) for x in every)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main(argv: list[str] | None = None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--sizes-mb", type=int, nargs="*", default=[1, 4, 16, 64, 256, 1024])
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--mirror", action="store_true", help="also write the bf16 mirror in the all-reduce kernel")
    ap.add_argument("--ag-gemm", action="store_true", help="also time the all-gather fused into the expert-bank GEMMs")
    ap.add_argument("--gather-rings", type=str, nargs="*", default=["8192x4x1", "8192x2x4", "4096x2x4"],
                    help="copy-ring shapes to time: chunk bytes x buffers per lane x copying lanes")
    a = ap.parse_args(argv)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    from nestor_b200.parallel import symm
    from nestor_b200.utils.distributed import init_distributed
    dev = init_distributed(True)
    if not dist.is_initialized():
        # a single rank (no launcher): the kernels then run their local leg only (flag round trip with itself, own
        # buffer read, scaled, written), which is the case a one-GPU profiler capture can take
        os.environ.setdefault("MASTER_PORT", "29655")
        dist.init_process_group("nccl", init_method="env://", world_size=1, rank=0, device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    nmax = max(a.sizes_mb) * 1024 * 1024 // 4
    g = symm.symmetric_empty(nmax, torch.float32, dev)
    g.copy_(torch.randn(nmax, device=dev) * 1e-3)
    mirror = symm.symmetric_empty(nmax, torch.bfloat16, dev) if a.mirror else None
    # correctness first: same result as NCCL
    ref = g.clone()
    dist.all_reduce(ref)
    ref /= world
    first = symm.FusedAllReduce(g, [(0, nmax)], mirror)
    first.run(1.0 / world)
    torch.cuda.synchronize()
    err = (g - ref).abs().max().item()
    have_nvls = first.group.nvls
    if rank == 0:
        print(f"world {world}: fused all-reduce max |diff| vs NCCL = {err:.2e}; NVLink multicast mapping: "
              f"{'yes' if have_nvls else 'no'}", flush=True)

    def both(make):
        """Time one collective on plain peer loads/stores and, when the buffers have a multicast mapping, on multimem."""
        out = {}
        for name, env in (("p2p", "0"), ("nvls", "auto")):
            if name == "nvls" and not have_nvls:
                continue
            os.environ["NESTOR_B200_NVLS"] = env
            obj, fn = make()
            out[name] = timed(fn, a.reps, dev)
            obj.group.check()
        os.environ["NESTOR_B200_NVLS"] = "auto"
        return out

    for mb in a.sizes_mb:
        n = mb * 1024 * 1024 // 4
        t = g[:n].clone()

        def make_ar():
            fa = symm.FusedAllReduce(g, [(0, n)], mirror)
            return fa, lambda: fa.run(1.0 / world)

        res = both(make_ar)
        ms_nccl = timed(lambda: dist.all_reduce(t), a.reps, dev)
        bus = 2 * (world - 1) / world * n * 4 / 1e9
        if rank == 0:
            ours = " | ".join(f"{k} {v:8.3f} ms {bus / v * 1e3:6.0f} GB/s bus ({bus / v * 1e3 / PEER_COPY_GBS:5.1%} of the peer-copy rate)"
                              for k, v in res.items())
            print(f"all-reduce {mb:5d} MB: {ours} | NCCL {ms_nccl:8.3f} ms {bus / ms_nccl * 1e3:6.0f} GB/s", flush=True)
    # reduce-scatter onto ownership ranges (what the sharded optimizer uses) vs NCCL reduce_scatter_tensor
    for mb in a.sizes_mb:
        n = (mb * 1024 * 1024 // 4) // (4 * world) * (4 * world)
        per = n // world
        t = g[:n].clone()
        shard = torch.empty(per, dtype=torch.float32, device=dev)

        def make_rs():
            rs = symm.FusedReduceScatter(g)
            return rs, lambda: rs.run(rank * per, (rank + 1) * per, 1.0 / world)

        res = both(make_rs)
        ms_nccl = timed(lambda: dist.reduce_scatter_tensor(shard, t), a.reps, dev)
        bus = (world - 1) / world * n * 4 / 1e9
        if rank == 0:
            ours = " | ".join(f"{k} {v:8.3f} ms {bus / v * 1e3:6.0f} GB/s bus ({bus / v * 1e3 / PEER_COPY_GBS:5.1%})" for k, v in res.items())
            print(f"reduce-scatter {mb:5d} MB: {ours} | NCCL {ms_nccl:8.3f} ms {bus / ms_nccl * 1e3:6.0f} GB/s", flush=True)
    # parameter push vs all-gather + cast
    master = symm.symmetric_empty(nmax, torch.float32, dev)
    comp = symm.symmetric_empty(nmax, torch.bfloat16, dev)
    master.fill_(float(rank + 1))
    for mb in a.sizes_mb:
        n = (mb * 1024 * 1024 // 4) // (4 * world) * (4 * world)
        per = n // world

        def make_pp():
            pp = symm.ParamPush(master, comp, push_master=True)
            return pp, lambda: pp.run(rank * per, (rank + 1) * per)

        def make_pp_bf16():
            pp = symm.ParamPush(master, comp, push_master=False)
            return pp, lambda: pp.run(rank * per, (rank + 1) * per)

        res = both(make_pp)
        res16 = both(make_pp_bf16)
        shard = master[rank * per : (rank + 1) * per].clone()
        full = torch.empty(n, dtype=torch.float32, device=dev)
        ms_nccl = timed(lambda: (dist.all_gather_into_tensor(full, shard), full.to(torch.bfloat16)), a.reps, dev)
        bus = (world - 1) / world * n * 6 / 1e9          # fp32 master + bf16 compute copy cross the links
        if rank == 0:
            ours = " | ".join(f"{k} {v:8.3f} ms {bus / v * 1e3:6.0f} GB/s ({bus / v * 1e3 / PEER_COPY_GBS:5.1%} of the peer-copy rate)"
                              for k, v in res.items())
            print(f"param push {mb:5d} MB: {ours} | NCCL all-gather + cast {ms_nccl:8.3f} ms", flush=True)
            bus16 = (world - 1) / world * n * 2 / 1e9       # the bf16 compute copy alone crosses the links
            ours16 = " | ".join(f"{k} {v:8.3f} ms {bus16 / v * 1e3:6.0f} GB/s" for k, v in res16.items())
            print(f"param push {mb:5d} MB, compute copy only (what the training step uses): {ours16}", flush=True)
    if a.ag_gemm:
        bench_ag_gemm(dev, rank, world, a.reps, a.gather_rings)
    # leave in step: nothing of a rank is unmapped while a peer may still touch it
    torch.cuda.synchronize()
    dist.barrier()
    del g, mirror, master, comp, first
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()


def bench_ag_gemm(dev, rank: int, world: int, reps: int, rings: list[str]) -> None:
    """All-gather fused into the expert-bank GEMMs of nestor_200m against NCCL all-gather followed by the GEMM.

    Shapes: 98,304 dispatched rows over 64 experts, up||gate + SwiGLU ``[640 -> 2 x 216]`` and down
    ``[216 -> 640]``. Each rank owns 64 / W experts of every bank. The roofline is the slower of the product
    alone (timed here) and the remote bytes over the measured peer-copy rate.
    """

    from nestor_b200.ops import gemm as G
    from nestor_b200.parallel import symm
    E, d, h, rows = 64, 640, 216, 98304
    n = E * d * h
    per = E // world
    arena = symm.symmetric_empty(3 * n, torch.bfloat16, dev)
    arena.copy_(torch.randn(3 * n, device=dev) * 0.03)
    handle = symm.rendezvous(arena)
    vg, vu, vd = arena[:n].view(E, d, h), arena[n : 2 * n].view(E, d, h), arena[2 * n :].view(E, h, d)
    X = torch.randn(rows, d, device=dev).bfloat16()
    Hh = torch.randn(rows, h, device=dev).bfloat16()
    off = (torch.arange(E + 1, device=dev, dtype=torch.int32) * (rows // E)).contiguous()
    H, Gt, Ut = (G.rows_buffer(rows, h, torch.bfloat16, dev) for _ in range(3))
    Y = torch.empty(rows, d, dtype=torch.bfloat16, device=dev)
    stage = torch.empty(2 * n, dtype=torch.bfloat16, device=dev)
    flags = torch.zeros(257, dtype=torch.int32, device=dev)
    full = torch.empty(2 * n, dtype=torch.bfloat16, device=dev)
    shard_gu = torch.cat([vg[rank * per : (rank + 1) * per].reshape(-1), vu[rank * per : (rank + 1) * per].reshape(-1)]).clone()
    shard_d = vd[rank * per : (rank + 1) * per].reshape(-1).clone()
    torch.cuda.synchronize()
    dist.barrier()

    def up(gather, wg=vg, wu=vu):
        G.gemm_rows(X, wg, B2=wu, offsets=off, groups=E, b_mn=True, out=H, epilogue=G.SWIGLU, extra_out=(Gt, Ut), gather=gather)

    def down(gather, wd=vd):
        G.gemm_rows(Hh, wd, offsets=off, groups=E, b_mn=True, out=Y, gather=gather)

    def nccl_up():
        dist.all_gather_into_tensor(full, shard_gu)
        up(None)

    def nccl_down():
        dist.all_gather_into_tensor(full[:n], shard_d)
        down(None)

    base_up, base_down = timed(lambda: up(None), reps, dev), timed(lambda: down(None), reps, dev)
    t_nccl_up, t_nccl_down = timed(nccl_up, reps, dev), timed(nccl_down, reps, dev)
    remote_up, remote_down = 2 * n * 2 * (world - 1) / world, n * 2 * (world - 1) / world
    if rank == 0:
        print(f"all-gather + GEMM, world {world}: product alone up||gate {base_up * 1e3:.0f} us, down {base_down * 1e3:.0f} us; "
              f"NCCL all-gather then product {t_nccl_up * 1e3:.0f} / {t_nccl_down * 1e3:.0f} us; remote bytes "
              f"{remote_up / 1e6:.1f} / {remote_down / 1e6:.1f} MB = {remote_up / PEER_COPY_GBS / 1e3:.0f} / "
              f"{remote_down / PEER_COPY_GBS / 1e3:.0f} us at the peer-copy rate", flush=True)
    for ring in rings:
        chunk, nbuf, lanes = (int(v) for v in ring.split("x"))
        spec = G.Gather(src=[int(handle.buffer_ptrs[r]) for r in range(world)], arena_ptr=arena.data_ptr(), stage=stage,
                        flags=flags, groups_per_rank=per, chunk=chunk, nbuf=nbuf, lanes=lanes)
        r_up, r_down = [], []
        t_up, t_down = timed(lambda: up(spec), reps, dev, r_up), timed(lambda: down(spec), reps, dev, r_down)
        roof_up = max(base_up, remote_up / PEER_COPY_GBS / 1e6)
        roof_down = max(base_down, remote_down / PEER_COPY_GBS / 1e6)
        if rank == 0:
            print(f"  fused, copy ring {ring:>9s}: up||gate {t_up * 1e3:.0f} us ({roof_up / t_up:5.1%} of roofline), "
                  f"down {t_down * 1e3:.0f} us ({roof_down / t_down:5.1%}); per rank "
                  f"{'/'.join(f'{x * 1e3:.0f}' for x in r_up)} and {'/'.join(f'{x * 1e3:.0f}' for x in r_down)} us", flush=True)
    from nestor_b200.ops import _lib
    torch.cuda.synchronize()
    _lib.check_status(dev)


if __name__ == "__main__":
    main()
