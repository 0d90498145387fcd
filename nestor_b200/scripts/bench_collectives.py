"""Micro-benchmark of the in-kernel collectives against NCCL (gradient all-reduce + cast, parameter push).

``torchrun --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 -m nestor_b200.scripts.bench_collectives``
times, for 1 MB ... 1 GB fp32 buffers: the owner-push all-reduce kernel (fp32 sum, 1/W scale, optional bf16
mirror) and ``torch.distributed.all_reduce`` (NCCL) on the same buffer, and the parameter push (all-gather fused
with the bf16 cast) against ``all_gather_into_tensor`` + cast. Device-timed with CUDA events, max over ranks.
Bus bandwidth is ``2 (W-1)/W * bytes / time`` for the all-reduce and ``(W-1)/W * bytes / time`` for the
gather; the roofline is the measured peer copy of 770 GB/s per direction per GPU (900 nominal).
"""

from __future__ import annotations

import argparse
import os

import torch
import torch.distributed as dist

PEER_COPY_GBS = 770.0


def timed(fn, reps: int, dev) -> float:
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
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main(argv: list[str] | None = None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--sizes-mb", type=int, nargs="*", default=[1, 4, 16, 64, 256, 1024])
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--mirror", action="store_true", help="also write the bf16 mirror in the all-reduce kernel")
    a = ap.parse_args(argv)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    from nestor_b200.parallel import symm
    from nestor_b200.utils.distributed import init_distributed
    dev = init_distributed(True)
    rank, world = dist.get_rank(), dist.get_world_size()
    nmax = max(a.sizes_mb) * 1024 * 1024 // 4
    g = symm.symmetric_empty(nmax, torch.float32, dev)
    g.copy_(torch.randn(nmax, device=dev) * 1e-3)
    mirror = symm.symmetric_empty(nmax, torch.bfloat16, dev) if a.mirror else None
    # correctness first: same result as NCCL
    ref = g.clone()
    dist.all_reduce(ref)
    ref /= world
    symm.FusedAllReduce(g, [(0, nmax)], mirror).run(1.0 / world)
    torch.cuda.synchronize()
    err = (g - ref).abs().max().item()
    if rank == 0:
        print(f"world {world}: fused all-reduce max |diff| vs NCCL = {err:.2e}", flush=True)
    for mb in a.sizes_mb:
        n = mb * 1024 * 1024 // 4
        fa = symm.FusedAllReduce(g, [(0, n)], mirror)
        t = g[:n].clone()
        ms = timed(lambda: fa.run(1.0 / world), a.reps, dev)
        ms_nccl = timed(lambda: dist.all_reduce(t), a.reps, dev)
        bus = 2 * (world - 1) / world * n * 4 / 1e9
        if rank == 0:
            print(f"all-reduce {mb:5d} MB: fused {ms:8.3f} ms {bus / ms * 1e3:6.0f} GB/s bus "
                  f"({bus / ms * 1e3 / PEER_COPY_GBS:5.1%} of the peer-copy rate) | NCCL {ms_nccl:8.3f} ms "
                  f"{bus / ms_nccl * 1e3:6.0f} GB/s", flush=True)
        fa.group.check()
    # parameter push vs all-gather + cast
    master = symm.symmetric_empty(nmax, torch.float32, dev)
    comp = symm.symmetric_empty(nmax, torch.bfloat16, dev)
    master.fill_(float(rank + 1))
    pp = symm.ParamPush(master, comp)
    for mb in a.sizes_mb:
        n = (mb * 1024 * 1024 // 4) // (4 * world) * (4 * world)
        per = n // world
        ms = timed(lambda: pp.run(rank * per, (rank + 1) * per), a.reps, dev)
        shard = master[rank * per : (rank + 1) * per].clone()
        full = torch.empty(n, dtype=torch.float32, device=dev)
        ms_nccl = timed(lambda: (dist.all_gather_into_tensor(full, shard), full.to(torch.bfloat16)), a.reps, dev)
        bus = (world - 1) / world * n * 6 / 1e9          # fp32 master + bf16 compute copy cross the links
        if rank == 0:
            print(f"param push {mb:5d} MB: fused {ms:8.3f} ms {bus / ms * 1e3:6.0f} GB/s "
                  f"({bus / ms * 1e3 / PEER_COPY_GBS:5.1%} of the peer-copy rate) | NCCL all-gather + cast {ms_nccl:8.3f} ms", flush=True)
        pp.group.check()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
