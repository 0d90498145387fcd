"""Shared pytest setup: the ``gpu`` marker and a few helpers."""

import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

os.environ.setdefault("WANDB_MODE", "disabled")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture
def tiny_scale(monkeypatch):
    """Register a small 'tiny' rung on the pretraining tables (d=128) for fast model tests."""

    from nestor_b200.experiments import pretrain as P

    monkeypatch.setitem(P.SCALES, "tiny", P.Scale("tiny", 128, 4, 8, 512, 10, 2, 1024))
    monkeypatch.setitem(P.NESTOR_LAYERS, "tiny", (2, 1, 1, 1, 1, 1, 2))
    monkeypatch.setitem(P.NESTOR_PRIVATE_EXPERTS, "tiny", 3)
    monkeypatch.setattr(P, "NESTOR_MIN_PRIVATE_WIDTH", 24)
    for fam in ("dense", "moe", "nestor"):
        monkeypatch.setitem(P.BATCH_SHAPE, (fam, "tiny"), (2, 1))
    monkeypatch.setenv("DCLM_BLOCK_SIZE", "64")
    return P
