"""Dump the CUDA caching-allocator history once when the process first runs out of device memory.

``install_oom_snapshot(run_dir, rank)`` starts allocator history recording and registers an
out-of-memory observer that writes ``<run_dir>/diag_oom_rank<r>.pickle`` the first time an
allocation fails (later failures are ignored; ``suspended`` mutes it around deliberate probing such
as batch-size calibration). Armed by ``NESTOR_DIAG_OOM_SNAPSHOT=1``. Reference:
``nestor/train/oom_snapshot.py:36-133``.
"""

from __future__ import annotations

import pickle
from pathlib import Path

import torch


class OomSnapshotDumper:
    def __init__(self, path: Path) -> None:
        self.path = Path(path)
        self.dumped = False
        self.suspended = False

    def __call__(self, device: int, alloc: int, device_alloc: int, device_free: int) -> None:
        if self.dumped or self.suspended:
            return
        self.dumped = True
        try:
            snap = torch.cuda.memory._snapshot()
            self.path.parent.mkdir(parents=True, exist_ok=True)
            with open(self.path, "wb") as f:
                pickle.dump({"snapshot": snap, "requested_bytes": alloc, "device_free": device_free}, f)
        except Exception:   # diagnostics must never mask the original error
            pass


def install_oom_snapshot(run_dir: Path, rank: int = 0, max_entries: int = 100_000) -> OomSnapshotDumper | None:
    if not torch.cuda.is_available():
        return None
    dumper = OomSnapshotDumper(Path(run_dir) / f"diag_oom_rank{rank}.pickle")
    try:
        torch.cuda.memory._record_memory_history(max_entries=max_entries)
        torch._C._cuda_attach_out_of_memory_observer(dumper)
    except Exception:
        return None
    return dumper
