"""Collective protocols among real gloo ranks on CPU (no GPU, no mocks): gradient averaging over the
arena, owner-sharded Muon against the unsharded optimizer, buffer synchronisation, consolidated
optimizer state, and host-side failure detection (a rank that never joins makes the collective of the
others fail within a short process-group timeout)."""

import datetime
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from torch import nn

from nestor_b200.configs import MuonAdamWConfig
from nestor_b200.models.tags import ADAMW_DECAY, muon_matrix, tag


def _collect(procs, q, n, timeout=240.0):
    """``n`` results from the workers' queue, without waiting forever on a worker that died or hangs."""

    import time
    results, deadline = [], time.monotonic() + timeout
    while len(results) < n:
        if not q.empty():
            results.append(q.get())
        elif any(p.exitcode not in (None, 0) for p in procs) or time.monotonic() > deadline:
            for p in procs:
                if p.is_alive():
                    p.terminate()
            raise AssertionError(f"workers failed or timed out (exit codes {[p.exitcode for p in procs]})")
        else:
            time.sleep(0.05)
    return results


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class Net(nn.Module):
    def __init__(self):
        super().__init__()
        torch.manual_seed(7)
        self.w1 = tag(nn.Parameter(torch.randn(16, 24) * 0.1), muon_matrix(16, 24))
        self.w2 = tag(nn.Parameter(torch.randn(16, 24) * 0.1), muon_matrix(16, 24))
        self.bank = tag(nn.Parameter(torch.randn(2, 24, 8) * 0.1), muon_matrix(8, 24))
        self.e = tag(nn.Parameter(torch.randn(10, 24) * 0.1), ADAMW_DECAY)
        self.register_buffer("choice_bias", torch.zeros(4))

    def loss(self, x):
        h = x @ self.e.t()
        return (h.sum() + ((x @ self.w1.t()) ** 2).sum() + ((x @ self.w2.t()) * 0.5).sum()
                + torch.einsum("nd,edh->neh", x, self.bank).pow(2).sum())


def _data(rank, step):
    g = torch.Generator().manual_seed(100 + 10 * step + rank)
    return torch.randn(5, 24, generator=g)


def _worker(rank, world, port, q, mode):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    os.environ["NESTOR_MUON_SHARD"] = "1" if mode == "sharded" else "0"
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=30))
    from nestor_b200.parallel.arena import ParamArena
    from nestor_b200.parallel.grad_sync import GradReducer
    from nestor_b200.train.optim import build_optimizer
    net = Net()
    arena = ParamArena(net)
    red = GradReducer(arena, transport="gloo", bucket_mb=1)
    opt = build_optimizer(MuonAdamWConfig(lr_muon=0.02, lr_adamw=1e-2, weight_decay=0.1), net)
    assert opt.sharded == (mode == "sharded")
    net.choice_bias.fill_(float(rank))
    red.sync_buffers(net)
    assert float(net.choice_bias[0]) == 0.0
    for step in range(3):
        arena.zero_grad()
        net.loss(_data(rank, step)).backward()
        red.reduce()
        opt.step()
    if mode == "sharded":
        opt.consolidate_state_dict(to=0)
    state = opt.state_dict() if rank == 0 else None
    q.put((rank, arena.master.clone().numpy(), None if state is None else len(state["state"]),
           sorted(opt.owner.values()) if mode == "sharded" else None))
    dist.barrier()
    dist.destroy_process_group()


def _single_process_reference(world):
    from nestor_b200.parallel.arena import ParamArena
    from nestor_b200.train.optim import build_optimizer
    net = Net()
    arena = ParamArena(net)
    opt = build_optimizer(MuonAdamWConfig(lr_muon=0.02, lr_adamw=1e-2, weight_decay=0.1), net, shard=False)
    for step in range(3):
        arena.zero_grad()
        for r in range(world):
            (net.loss(_data(r, step)) / world).backward()
        opt.step()
    return arena.master.clone().numpy()


@pytest.mark.parametrize("mode", ["replicated", "sharded"])
def test_two_ranks_match_the_single_process_run(mode):
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q, mode)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted(_collect(procs, q, world), key=lambda t: t[0])
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    want = _single_process_reference(world)
    for rank, master, n_state, owners in results:
        assert abs(master - want).max() < 2e-5, (mode, rank)
    assert results[0][2] == 4                               # rank 0's state dict covers every parameter
    if mode == "sharded":
        assert set(results[0][3]) == {0, 1}                 # both ranks own Muon parameters


def _lonely_rank(port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK="0", WORLD_SIZE="2")
    try:
        dist.init_process_group("gloo", rank=0, world_size=2, timeout=datetime.timedelta(seconds=3))
        dist.all_reduce(torch.ones(1))
        q.put("joined")
    except Exception as exc:
        q.put(type(exc).__name__)


def test_missing_rank_is_detected_by_timeout():
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    p = ctx.Process(target=_lonely_rank, args=(_free_port(), q))
    p.start()
    (outcome,) = _collect([p], q, 1, timeout=60.0)
    p.join(30)
    assert not p.is_alive()
    assert outcome != "joined"


# ------------------------------------------------------------------ the whole trainer on two ranks
def _tiny_job(accum):
    import dataclasses as dc
    from nestor_b200.experiments.tiny import nestor_tiny
    job = nestor_tiny().jobs[0]
    return dc.replace(job, grad_accum_steps=accum)


def _tokens(shard, step):
    g = torch.Generator().manual_seed(1000 + 10 * step + shard)
    return torch.randint(0, 100_277, (2, 64), generator=g)


def _quiet(trainer):
    trainer.model.train()
    for blk in trainer.model.backbone.blocks:      # no exploration noise: both runs must route identically
        blk.freeze_routing_noise = True


def _trainer_rank(rank, world, port, q, sharded):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      DCLM_BLOCK_SIZE="64", NESTOR_LOSSFREE_GLOBAL_COUNTS="1",
                      NESTOR_MUON_SHARD="1" if sharded else "0", WANDB_MODE="disabled")
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    from nestor_b200.models import Model
    from nestor_b200.train.trainer import Trainer
    torch.set_num_threads(1)                          # repeatable reductions: the comparison does not depend on scheduling
    torch.manual_seed(0)
    job = _tiny_job(1)
    tr = Trainer(job, Model.from_config(job.model), [], device=torch.device("cpu"))
    _quiet(tr)
    norms = []
    for step in range(2):
        ids = _tokens(rank, step)
        loss, counts = tr.train_step((ids, ids))
        norms.append(float(tr.update_weights(counts)))
    bias = torch.cat([r.choice_bias.flatten() for _, r in tr.model.backbone.routers()])
    q.put((rank, tr.arena.master.clone().numpy(), bias.numpy(), norms))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("sharded", [False, True])
def test_trainer_on_two_ranks_matches_accumulation_in_one_process(sharded, monkeypatch):
    """Two gloo ranks, one micro-batch each, against one process that accumulates the same two micro-batches: the
    gradient mean over ranks, the clipping norm, both optimizers (replicated, and with owner-sharded state), the
    parameter broadcast and the balancing-bias update from global counts leave every rank with the single-process
    weights and biases."""

    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    procs = [ctx.Process(target=_trainer_rank, args=(r, world, port, q, sharded)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted(_collect(procs, q, world), key=lambda t: t[0])
    for p in procs:
        p.join(120)
        assert p.exitcode == 0

    monkeypatch.setenv("DCLM_BLOCK_SIZE", "64")
    monkeypatch.setenv("NESTOR_LOSSFREE_GLOBAL_COUNTS", "1")
    from nestor_b200.models import Model
    from nestor_b200.models.nestor import add_router_counts
    from nestor_b200.train.trainer import Trainer
    threads = torch.get_num_threads()
    torch.set_num_threads(1)
    try:
        torch.manual_seed(0)
        job = _tiny_job(2)
        tr = Trainer(job, Model.from_config(job.model), [], device=torch.device("cpu"))
        _quiet(tr)
        start = tr.arena.master.clone().numpy()
        want_norms = []
        for step in range(2):
            total = None
            for shard in range(world):
                ids = _tokens(shard, step)
                loss, counts = tr.train_step((ids, ids))
                total = add_router_counts(total, counts)
            want_norms.append(float(tr.update_weights(total)))
    finally:
        torch.set_num_threads(threads)
    want = tr.arena.master.clone().numpy()
    want_bias = torch.cat([r.choice_bias.flatten() for _, r in tr.model.backbone.routers()]).numpy()
    assert abs(want_bias).max() > 0                      # the balancing update really moved the biases
    import numpy as np
    moved = np.linalg.norm(want - start)
    for rank, master, bias, norms in results:
        # (Newton-Schulz runs in bf16: a last-bit difference in a reduced gradient can flip a rounding inside it, which
        # moves single matrices by a percent or two of their update; the clipping norms below are the sharp check of
        # the reduced gradients, and the ranks must agree with each other exactly)
        assert np.linalg.norm(master - want) < 1e-2 * moved, (rank, np.linalg.norm(master - want), moved)
        assert abs(master - want).max() < 1e-3, (rank, abs(master - want).max())
        assert (bias == want_bias).all(), rank
        assert all(abs(a - b) < 1e-5 * max(1.0, abs(b)) for a, b in zip(norms, want_norms)), (norms, want_norms)
    assert (results[0][1] == results[1][1]).all()
