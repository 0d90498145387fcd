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
