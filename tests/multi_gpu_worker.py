"""Worker for the multi-GPU tests (launched with ``python -m torch.distributed.run``): checks the fused
all-reduce / reduce-scatter against NCCL and the parameter push, on plain peer loads/stores and (when the symmetric
buffers have an NVLink multicast mapping) on ``multimem`` instructions, then that replicas stay identical over
optimizer steps of the tiny model. Every rank leaves in step, after the symmetric buffers are released."""

import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
import torch
import torch.distributed as dist

from nestor_b200.ops import _lib
from nestor_b200.parallel import symm
from nestor_b200.utils.distributed import init_distributed


def check_gathered_gemm(dev, rank: int, world: int) -> None:
    """Grouped products whose weights are staged from their owner ranks inside the GEMM launch."""

    from nestor_b200.ops import gemm as G
    E, d, h, rows = 8, 640, 216, 6000
    torch.manual_seed(7)                       # the same values on every rank
    Wg, Wu = (torch.randn(E, d, h, device=dev) * 0.05).bfloat16(), (torch.randn(E, d, h, device=dev) * 0.05).bfloat16()
    X = torch.randn(rows, d, device=dev).bfloat16()
    off = torch.tensor([0, 700, 700, 1500, 2600, 3000, 4100, 5000, rows], dtype=torch.int32, device=dev)
    n = E * d * h
    arena = symm.symmetric_empty(2 * n + 64, torch.bfloat16, dev)
    arena.fill_(float("nan"))                  # a rank holds valid values for its own experts only
    per = E // world
    vg, vu = arena[64 : 64 + n].view(E, d, h), arena[64 + n : 64 + 2 * n].view(E, d, h)
    vg[rank * per : (rank + 1) * per] = Wg[rank * per : (rank + 1) * per]
    vu[rank * per : (rank + 1) * per] = Wu[rank * per : (rank + 1) * per]
    handle = symm.rendezvous(arena)
    torch.cuda.synchronize()
    dist.barrier()
    spec = G.Gather(src=[int(handle.buffer_ptrs[r]) for r in range(world)], arena_ptr=arena.data_ptr(),
                    stage=torch.full((2 * n,), float("nan"), device=dev, dtype=torch.bfloat16),
                    flags=torch.zeros(257, dtype=torch.int32, device=dev), groups_per_rank=per)

    def run(gather, wg, wu):
        H = torch.full((rows, h), float("nan"), device=dev, dtype=torch.bfloat16)
        Gt, Ut = torch.empty_like(H), torch.empty_like(H)
        G.gemm_rows(X, wg, B2=wu, offsets=off, groups=E, b_mn=True, out=H, epilogue=G.SWIGLU, extra_out=(Gt, Ut),
                    gather=gather)
        return H, G.gemm_rows(H, wg, offsets=off, groups=E, gather=gather)

    want = run(None, Wg, Wu)
    for _ in range(2):
        got = run(spec, vg, vu)
        torch.cuda.synchronize()
        _lib.check_status(dev)
        assert all(torch.equal(a, b) for a, b in zip(want, got)), "fused all-gather GEMM mismatch"
    dist.barrier()


def check_collectives(dev, rank: int, world: int, nvls: str) -> bool:
    """All-reduce, ragged reduce-scatter and parameter push against NCCL results; returns whether multimem was used."""

    os.environ["NESTOR_B200_NVLS"] = nvls
    N = 8 * 1024 * 1024
    g = symm.symmetric_empty(N, torch.float32, dev)
    g.copy_(torch.randn(N, device=dev) * 1e-3)
    ref = g.clone()
    dist.all_reduce(ref)
    ref /= world
    far = symm.FusedAllReduce(g, [(0, N // 2), (N // 2, N // 2)])
    dist.barrier()
    far.run(1.0 / world)
    torch.cuda.synchronize()
    far.group.check()
    assert (g - ref).abs().max().item() < 1e-6, "fused all-reduce mismatch"
    # reduce-scatter with ragged ownership ranges: every rank ends with the average of its own range only
    g.copy_(torch.randn(N, device=dev) * 1e-3)
    ref = g.clone()
    dist.all_reduce(ref)
    ref /= world
    cuts = [0] + [((N * (r + 1) // world) + 4096 * (r % 2)) // 4 * 4 for r in range(world - 1)] + [N]
    lo, hi = cuts[rank], cuts[rank + 1]
    mine = g.clone()
    frs = symm.FusedReduceScatter(g)
    dist.barrier()
    frs.run(lo, hi, 1.0 / world)
    torch.cuda.synchronize()
    frs.group.check()
    assert (g[lo:hi] - ref[lo:hi]).abs().max().item() < 1e-6, "fused reduce-scatter mismatch"
    assert torch.equal(g[:lo], mine[:lo]) and torch.equal(g[hi:], mine[hi:]), "reduce-scatter wrote outside its range"
    dist.barrier()
    M = 4 * 1024 * 1024
    master, comp = symm.symmetric_empty(M, torch.float32, dev), symm.symmetric_empty(M, torch.bfloat16, dev)
    master.fill_(float(rank + 1))
    comp.zero_()
    torch.cuda.synchronize()
    dist.barrier()
    per = M // world
    pp = symm.ParamPush(master, comp, push_master=False)      # the compute copy alone travels
    pp.run(rank * per, (rank + 1) * per)
    torch.cuda.synchronize()
    pp.group.check()
    dist.barrier()
    want = torch.arange(1, world + 1, device=dev, dtype=torch.float32).repeat_interleave(per)
    assert torch.equal(comp.float(), want), "parameter push (compute copy) mismatch"
    assert torch.equal(master, torch.full_like(master, float(rank + 1))), "a bf16-only push must not touch the masters"
    symm.gather_ranges(master, [r * per for r in range(world + 1)])
    assert torch.equal(master, want), "gather_ranges mismatch"
    master.fill_(float(rank + 1))
    comp.zero_()
    torch.cuda.synchronize()
    dist.barrier()
    pp = symm.ParamPush(master, comp, push_master=True)
    pp.run(rank * per, (rank + 1) * per)
    torch.cuda.synchronize()
    pp.group.check()
    dist.barrier()
    assert torch.equal(master, want) and torch.equal(comp.float(), want), "parameter push mismatch"
    used = bool(far.group.nvls and frs.group.nvls and pp.group.nvls)
    torch.cuda.synchronize()
    dist.barrier()
    del g, master, comp, far, frs, pp
    return used


def main() -> None:
    dev = init_distributed(True)
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.manual_seed(100 + rank)
    used = {mode: check_collectives(dev, rank, world, mode) for mode in ("0", "auto")}
    assert not used["0"], "NESTOR_B200_NVLS=0 must keep the collectives on plain peer loads and stores"
    if rank == 0:
        print(f"collectives ok on peer loads/stores; multimem path {'ok' if used['auto'] else 'not available on this box'}", flush=True)
    check_gathered_gemm(dev, rank, world)
    os.environ.setdefault("DCLM_DATA_PATH", "/tmp/unused.bin")
    from nestor_b200.experiments.tiny import nestor_tiny
    from nestor_b200.models import Model
    from nestor_b200.train.trainer import Trainer
    results = {}
    for zero in ("1", "0"):     # sharded optimizer state + reduce-scatter, then replicated AdamW + all-reduce
        os.environ["NESTOR_ZERO1"] = zero
        torch.manual_seed(0)
        job = nestor_tiny().jobs[0]
        tr = Trainer(job, Model.from_config(job.model), [], device=dev)
        assert tr.param_push is not None and tr.reducer.transport == "fused" and tr.zero == (zero == "1")
        tr.model.train()
        for step in range(3):
            torch.manual_seed(1000 + step * 10 + rank)
            ids = torch.randint(0, 100277, (2, 256), device=dev)
            loss, counts = tr.train_step((ids, ids))
            tr.update_weights(counts)
        torch.cuda.synchronize()
        _lib.check_status(dev)
        if zero == "1":
            # the push moved the bf16 copy only: a rank's masters outside its own range are stale until gathered
            assert tr.masters_sharded
            lo, hi = tr.optimizer.owned_range()
            assert torch.equal(tr.arena.master[lo:hi].bfloat16(), tr.arena.compute[lo:hi])
        tr.gather_masters()
        assert torch.equal(tr.arena.master.bfloat16(), tr.arena.compute), "compute copy is not the cast of the masters"
        chk = torch.tensor([tr.arena.master.double().sum().item(), tr.arena.compute.double().sum().item()], device=dev,
                           dtype=torch.float64)
        gathered = [torch.zeros_like(chk) for _ in range(world)]
        dist.all_gather(gathered, chk)
        assert all(torch.equal(x, gathered[0]) for x in gathered), "replicas diverged"
        results[zero] = tr.arena.master.clone()
        sd = None
        tr.optimizer.consolidate_state_dict()
        if rank == 0:
            sd = tr.optimizer.state_dict()
            assert len(sd["state"]) == sum(len(g["params"]) for g in sd["param_groups"]), "optimizer state incomplete"
        del tr
    # the two paths sum the clip norm in different orders (and an in-switch reduction fixes no order at all); the
    # Newton-Schulz iteration runs in bf16, where a last-bit difference of its input flips roundings, so the
    # parameters agree to bf16-iteration noise rather than to fp32 round-off
    rel = ((results["1"] - results["0"]).norm() / results["0"].norm()).item()
    assert rel < 5e-4, f"sharded and replicated optimizer paths disagree: {rel}"
    # expert banks read from their owner ranks through the all-gather fused into the bank GEMMs
    from nestor_b200.ops import cuda as cuda_ops
    os.environ["NESTOR_ZERO1"], os.environ["NESTOR_FSDP_BANKS"] = "1", "1"
    torch.manual_seed(0)
    job = nestor_tiny().jobs[0]
    tr = Trainer(job, Model.from_config(job.model), [], device=dev)
    assert cuda_ops.BANK_SHARDS is not None
    tr.model.train()
    for step in range(3):
        torch.manual_seed(1000 + step * 10 + rank)
        ids = torch.randint(0, 100277, (2, 256), device=dev)
        loss, counts = tr.train_step((ids, ids))
        tr.update_weights(counts)
    torch.cuda.synchronize()
    _lib.check_status(dev)
    assert cuda_ops.BANK_SHARDS.gathered_bytes > 0, "no bank product used the fused all-gather"
    tr.gather_masters()
    rel = ((tr.arena.master - results["1"]).norm() / results["1"].norm()).item()
    assert rel < 5e-4, f"rank-sharded banks disagree with replicated banks: {rel}"
    cuda_ops.BANK_SHARDS = None
    os.environ["NESTOR_FSDP_BANKS"] = "0"
    dist.barrier()
    torch.cuda.synchronize()
    dist.barrier()
    del tr, results
    torch.cuda.synchronize()
    dist.barrier()
    if rank == 0:
        print("MULTI_GPU_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
