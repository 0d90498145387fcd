"""Process-group control plane: init / teardown, rank helpers, small reductions.

The control plane is ``torch.distributed`` (NCCL on GPUs, gloo on CPU); the data plane
(gradient reduction, parameter distribution) lives in :mod:`nestor_b200.parallel`.
Reference behaviour: ``nestor/utils/distributed.py:18-88`` (env rendezvous, long timeout
so cold starts do not trip the watchdog: ``NESTOR_DIST_TIMEOUT_MIN``, default 90),
``:189-255`` (barrier / cleanup / summed reductions), ``:197`` (padded rank indices).
"""

from __future__ import annotations

import datetime
import os

import torch
import torch.distributed as dist


def dist_ready() -> bool:
    return dist.is_available() and dist.is_initialized()


def get_rank() -> int:
    return dist.get_rank() if dist_ready() else 0


def get_world_size() -> int:
    return dist.get_world_size() if dist_ready() else 1


def get_local_rank() -> int:
    return int(os.environ.get("LOCAL_RANK", "0"))


def is_main_process() -> bool:
    return get_rank() == 0


def init_distributed(enabled: bool = True, backend: str | None = None) -> torch.device:
    """Join the torchrun rendezvous if one is described in the environment; pick the device."""

    use_cuda = torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(get_local_rank())
        device = torch.device("cuda", get_local_rank())
    else:
        device = torch.device("cpu")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if enabled and world > 1 and not dist_ready():
        minutes = float(os.environ.get("NESTOR_DIST_TIMEOUT_MIN", "90"))
        kwargs = {}
        if use_cuda:
            kwargs["device_id"] = device
        dist.init_process_group(
            backend=backend or ("nccl" if use_cuda else "gloo"), init_method="env://",
            timeout=datetime.timedelta(minutes=minutes), **kwargs)
    return device


def barrier() -> None:
    if dist_ready() and get_world_size() > 1:
        dist.barrier()


def cleanup_distributed() -> None:
    if dist_ready():
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def sum_tensor_across_ranks(t: torch.Tensor) -> torch.Tensor:
    if dist_ready() and get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return t


def max_across_ranks(value: float, device: torch.device) -> float:
    t = torch.tensor([value], dtype=torch.float64, device=device if device.type == "cuda" else "cpu")
    if dist_ready() and get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def get_padded_rank_indices(n: int, rank: int | None = None, world: int | None = None) -> list[int]:
    """Indices of this rank's share of ``n`` items, padded by wrap-around so all ranks get equal counts."""

    rank = get_rank() if rank is None else rank
    world = get_world_size() if world is None else world
    per = (n + world - 1) // world
    idx = list(range(n))
    idx += idx[: per * world - n] if n else []
    return idx[rank : per * world : world]
