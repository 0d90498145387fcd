"""Flat token ``.bin`` datasets and a pinned-memory window loader.

``DclmTokenDataset`` has the reference's contract (``nestor/data/datasets.py:70-167``): the
file is one contiguous token array (dtype from the ``.meta.json`` sidecar, else the config),
served as non-overlapping ``block_size`` windows with an optional id remap; there is no
document masking, and an item is ``(window, window.clone())`` as int64.

``PinnedWindowLoader`` replaces the worker-process ``DataLoader`` for the training loop:
a background thread gathers each micro-batch's windows straight from the memory map into
a ring of page-locked staging buffers (numpy slicing releases the GIL), so the training
thread only issues one asynchronous host-to-device copy per micro-batch. Ordering is the
``DistributedSampler`` permutation (seeded by epoch), so resume fast-forward and the
seen-subset tooling see the same window sequence as a stock sampler would produce.
"""

from __future__ import annotations

import json
import queue
import threading
from pathlib import Path
from typing import Iterator

import numpy as np
import torch
from torch.utils.data import Dataset

from nestor_b200.configs import DataLoaderConfig, DatasetConfig, DclmDatasetConfig


class DclmTokenDataset(Dataset):
    def __init__(self, config: DclmDatasetConfig) -> None:
        self.config = config
        path = Path(config.data_path)
        if not path.is_file():
            raise FileNotFoundError(f"Token file not found: {path}. Run scripts/preprocess_dclm.py to produce it.")
        dtype_name = config.token_dtype
        meta_path = path.with_suffix(path.suffix + ".meta.json")
        meta: dict = json.loads(meta_path.read_text()) if meta_path.is_file() else {}
        dtype_name = str(meta.get("token_dtype", dtype_name))
        self.tokens = np.memmap(path, dtype=np.dtype(dtype_name), mode="r")
        self.num_tokens = int(self.tokens.shape[0])
        if isinstance(meta.get("num_tokens"), int) and meta["num_tokens"] != self.num_tokens:
            raise ValueError(f"meta num_tokens {meta['num_tokens']} != {self.num_tokens} implied by the file size.")
        self.block_size = config.block_size
        self.num_windows = self.num_tokens // self.block_size
        if self.num_windows == 0:
            raise ValueError(f"Corpus has {self.num_tokens} tokens, fewer than one block of {self.block_size}.")
        self.remap = dict(config.token_remap)

    def __len__(self) -> int:
        return self.num_windows

    def read_into(self, index: int, out: np.ndarray) -> None:
        """Copy window ``index`` into ``out`` (int64, length ``block_size``), applying the remap."""

        a = index * self.block_size
        out[:] = self.tokens[a : a + self.block_size]
        for src, dst in self.remap.items():
            out[out == src] = dst

    def __getitem__(self, index: int) -> tuple[torch.Tensor, torch.Tensor]:
        buf = np.empty(self.block_size, dtype=np.int64)
        self.read_into(index, buf)
        block = torch.from_numpy(buf)
        return block, block.clone()


def build_dataset(config: DatasetConfig) -> Dataset:
    if isinstance(config, DclmDatasetConfig):
        return DclmTokenDataset(config)
    raise TypeError(f"Unknown dataset config {type(config).__name__}.")


def write_synthetic_bin(path: Path, num_tokens: int, vocab: int, seed: int = 0, *,
                        doc_len_range: tuple[int, int] | None = None, eot: int = 100257) -> Path:
    """Write a uniform-random token ``.bin`` (+ sidecar); optionally cut into log-uniform-length documents."""

    rng = np.random.default_rng(seed)
    tokens = rng.integers(0, min(vocab, eot), size=num_tokens, dtype=np.uint32)
    if doc_len_range is not None:
        lo, hi = doc_len_range
        at = 0
        while at < num_tokens:
            at += int(np.exp(rng.uniform(np.log(lo), np.log(hi))))
            if at - 1 < num_tokens:
                tokens[at - 1] = eot
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    tokens.tofile(path)
    Path(f"{path}.meta.json").write_text(json.dumps(
        {"token_dtype": "uint32", "num_tokens": int(num_tokens), "eot_token": eot, "synthetic": True}))
    return path


def epoch_permutation(n: int, epoch: int, seed: int, world: int, rank: int, shuffle: bool,
                      drop_last: bool = True) -> np.ndarray:
    """This rank's window indices for one epoch — the ``DistributedSampler`` rule.

    ``torch.randperm(n, generator=seed+epoch)`` truncated to a multiple of ``world`` (drop-last
    semantics) and strided by rank, so any tool that replays a stock sampler sees the same order.
    """

    if shuffle:
        g = torch.Generator()
        g.manual_seed(seed + epoch)
        order = torch.randperm(n, generator=g).numpy()
    else:
        order = np.arange(n)
    if drop_last:
        order = order[: (n // world) * world]
    else:
        pad = (-len(order)) % world
        order = np.concatenate([order, order[:pad]])
    return order[rank::world]


class PinnedWindowLoader:
    """Micro-batch iterator over a :class:`DclmTokenDataset` with pinned staging + prefetch thread.

    Yields ``(inputs, targets)`` int64 CPU tensors of shape ``[per_rank_batch, block_size]`` that
    live in page-locked memory. A yielded buffer stays untouched until ``depth`` further batches have been drawn
    (the ring holds ``2 * depth + 2`` buffers: ``depth`` queued, one being filled, one being handed over, ``depth``
    still owned by the consumer), so a consumer that copies asynchronously has to make sure that the copy of batch
    ``i`` has executed before it draws batch ``i + depth`` (``Trainer`` bounds its run-ahead to three batches).
    ``config.batch_size`` is the global batch; each rank takes ``batch_size // world``.
    """

    def __init__(self, dataset: DclmTokenDataset, config: DataLoaderConfig, *, rank: int = 0, world: int = 1,
                 seed: int = 0, depth: int = 4, pin: bool | None = None) -> None:
        if config.batch_size % world:
            raise ValueError(f"global batch {config.batch_size} is not divisible by world size {world}.")
        self.dataset, self.config = dataset, config
        self.rank, self.world, self.seed = rank, world, seed
        self.per_rank = config.batch_size // world
        self.epoch = 0
        self.depth = max(2, depth)
        pin = (config.pin_memory and torch.cuda.is_available()) if pin is None else pin
        self._ring = [torch.empty(self.per_rank, dataset.block_size, dtype=torch.int64,
                                  pin_memory=pin) for _ in range(2 * self.depth + 2)]

    def set_epoch(self, epoch: int) -> None:
        self.epoch = epoch

    def __len__(self) -> int:
        per_rank_windows = len(self.dataset) // self.world if self.config.drop_last else -(-len(self.dataset) // self.world)
        return per_rank_windows // self.per_rank if self.config.drop_last else -(-per_rank_windows // self.per_rank)

    def __iter__(self) -> Iterator[tuple[torch.Tensor, torch.Tensor]]:
        order = epoch_permutation(len(self.dataset), self.epoch, self.seed, self.world, self.rank,
                                  self.config.shuffle, self.config.drop_last)
        nb = len(self)
        q: queue.Queue = queue.Queue(maxsize=self.depth)
        stop = threading.Event()

        def produce() -> None:
            try:
                for b in range(nb):
                    if stop.is_set():
                        return
                    buf = self._ring[b % len(self._ring)]
                    arr = buf.numpy()
                    rows = order[b * self.per_rank : (b + 1) * self.per_rank]
                    for r, w in enumerate(rows):
                        self.dataset.read_into(int(w), arr[r])
                    if len(rows) < self.per_rank:
                        buf = buf[: len(rows)]
                    q.put(buf)
                q.put(None)
            except BaseException as exc:  # surface loader failures in the training thread
                q.put(exc)

        t = threading.Thread(target=produce, daemon=True, name="nestor-window-loader")
        t.start()
        try:
            while True:
                item = q.get()
                if item is None:
                    return
                if isinstance(item, BaseException):
                    raise item
                yield item, item
        finally:
            stop.set()
            while not q.empty():
                try:
                    q.get_nowait()
                except queue.Empty:
                    break
