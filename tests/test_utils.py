"""Small utilities: rank-padded index shares, metric logging (rank 0, wandb mirror), seeding, single-process fallbacks
of the collective helpers."""

import logging
import random

import numpy as np
import pytest
import torch

from nestor_b200.utils import distributed as D
from nestor_b200.utils import logging as L
from nestor_b200.utils.seed import set_seed


@pytest.mark.parametrize("n,world", [(10, 4), (8, 4), (3, 4), (0, 2), (7, 1)])
def test_padded_rank_shares_cover_everything_with_equal_counts(n, world):
    shares = [D.get_padded_rank_indices(n, r, world) for r in range(world)]
    per = (n + world - 1) // world
    assert all(len(s) == per for s in shares)                       # every rank gets the same count
    assert set(i for s in shares for i in s) == set(range(n))       # nothing is left out
    flat = [i for s in shares for i in s]
    assert len(flat) - len(set(flat)) == per * world - n            # padding repeats items from the front only


def test_single_process_fallbacks():
    assert D.get_rank() == 0 and D.get_world_size() == 1 and D.is_main_process() and not D.dist_ready()
    D.barrier(); D.cleanup_distributed()                            # no group: both are no-ops
    t = torch.tensor([3.0])
    assert D.sum_tensor_across_ranks(t) is t and float(t) == 3.0
    assert D.max_across_ranks(2.5, torch.device("cpu")) == 2.5
    assert D.init_distributed(enabled=True).type in ("cpu", "cuda")   # WORLD_SIZE unset: nothing to join


def test_metrics_go_to_the_console_and_the_tracker(monkeypatch):
    records = []

    class Capture(logging.Handler):
        def emit(self, record):
            records.append(record.getMessage())

    logger = L.get_logger("nestor_b200.test_metrics")
    logger.addHandler(Capture())
    sent = []

    class Run:
        def log(self, payload, step):
            sent.append((payload, step))

    L.set_wandb_run(Run())
    try:
        L.log_metrics(logger, {"loss": 1.23456789, "tokens": 42}, step=7, prefix="train/")
        assert records[-1] == "step 7 | loss=1.2346 tokens=42"
        assert sent == [({"train/loss": 1.23456789, "train/tokens": 42}, 7)]
        monkeypatch.setattr(L, "is_main_process", lambda: False)     # other ranks stay silent
        L.log_metrics(logger, {"loss": 9.0}, step=8)
        assert len(records) == 1 and len(sent) == 1
    finally:
        L.set_wandb_run(None)


def test_seed_covers_every_generator(monkeypatch):
    set_seed(11, rank_offset=2)
    a = (random.random(), float(np.random.rand()), float(torch.rand(())))
    set_seed(13)
    b = (random.random(), float(np.random.rand()), float(torch.rand(())))
    assert a == b                                                    # seed + rank offset is what counts
    set_seed(14)
    assert (random.random(), float(np.random.rand()), float(torch.rand(()))) != a
    assert torch.get_float32_matmul_precision() == "high"
    monkeypatch.setenv("NESTOR_DETERMINISTIC", "1")
    set_seed(1)
    assert torch.backends.cudnn.deterministic and not torch.backends.cudnn.benchmark
    monkeypatch.delenv("NESTOR_DETERMINISTIC")
    torch.backends.cudnn.deterministic = False
    set_seed(1)
    assert torch.backends.cudnn.benchmark


def test_supervised_batches_in_every_accepted_form():
    from nestor_b200.utils.batches import split_supervised_batch
    x, y = torch.arange(6).view(2, 3), torch.arange(6).view(2, 3) + 1
    for batch in ((x, y), [x, y], {"inputs": x, "targets": y}, {"inputs": x, "labels": y}, {"x": x, "y": y, "meta": 1}):
        a, b = split_supervised_batch(batch)
        assert a is x and b is y
    assert split_supervised_batch((["text a", "text b"], y))[0] == ["text a", "text b"]   # inputs may be anything
    for bad in ((x, y, x), {"inputs": x}, {"a": x, "b": y}, x, (x, [1, 2])):
        with pytest.raises(TypeError):
            split_supervised_batch(bad)


def test_trainer_accepts_mapping_batches(monkeypatch):
    from nestor_b200.experiments.tiny import nestor_tiny
    from nestor_b200.models import Model
    from nestor_b200.train.trainer import Trainer
    monkeypatch.setenv("DCLM_BLOCK_SIZE", "64")
    torch.manual_seed(0)
    job = nestor_tiny().jobs[0]
    tr = Trainer(job, Model.from_config(job.model), [], device=torch.device("cpu"))
    tr.model.eval(); tr.model.training = True
    for blk in tr.model.backbone.blocks:
        blk.freeze_routing_noise = True
    ids = torch.randint(0, 100_277, (2, 64))
    a, _ = tr.train_step((ids, ids))
    tr.arena.zero_grad()
    b, _ = tr.train_step({"inputs": ids, "labels": ids})
    assert float(a.total) == float(b.total)
