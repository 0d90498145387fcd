"""Per-token loss of long sequences without ever materialising ``[S, V]`` logits.

``sequence_nll`` runs the backbone once over a ``[1, S]`` sequence and applies the head in chunks of
``head_chunk`` targets; ``token_nll`` scores one target range. ``PerPositionLoss`` accumulates
losses by position over many documents and reports the mean-by-position curve, a NaN-aware moving
average and binned means. Reference: ``nestor/eval/long_context.py:27-250``.
"""

from __future__ import annotations

from typing import Any

import numpy as np
import torch
import torch.nn.functional as F
from torch import Tensor


def _hidden(model: Any, tokens: Tensor) -> tuple[Tensor, dict]:
    was = model.fused_head
    model.fused_head = True          # the model then returns the normalised head input
    try:
        out = model(tokens)
    finally:
        model.fused_head = was
    return out.pred, out.aux


def _head_logits(model: Any, hidden: Tensor) -> Tensor:
    cd = hidden.dtype
    return model.head(hidden, cd)


@torch.no_grad()
def token_nll(model: Any, tokens: Tensor, *, target_start: int, target_end: int) -> tuple[Tensor, dict]:
    if tokens.dim() != 2 or tokens.shape[0] != 1:
        raise ValueError(f"tokens must have shape (1, seq_len), got {tuple(tokens.shape)}")
    S = tokens.shape[1]
    if not 1 <= target_start < target_end <= S:
        raise ValueError(f"need 1 <= target_start < target_end <= seq_len, got {target_start}, {target_end}, {S}")
    hidden, aux = _hidden(model, tokens)
    logits = _head_logits(model, hidden[0, target_start - 1 : target_end - 1])
    return F.cross_entropy(logits.float(), tokens[0, target_start:target_end], reduction="none"), aux


@torch.no_grad()
def sequence_nll(model: Any, tokens: Tensor, *, head_chunk: int = 4096) -> tuple[Tensor, dict]:
    if tokens.dim() != 2 or tokens.shape[0] != 1 or tokens.shape[1] < 2:
        raise ValueError(f"tokens must have shape (1, seq_len >= 2), got {tuple(tokens.shape)}")
    if head_chunk < 1:
        raise ValueError(f"head_chunk must be >= 1, got {head_chunk}")
    S = tokens.shape[1]
    hidden, aux = _hidden(model, tokens)
    pieces = []
    for a in range(1, S, head_chunk):
        b = min(a + head_chunk, S)
        logits = _head_logits(model, hidden[0, a - 1 : b - 1])
        pieces.append(F.cross_entropy(logits.float(), tokens[0, a:b], reduction="none"))
    return torch.cat(pieces), aux


def moving_average(values: np.ndarray, window: int = 101) -> np.ndarray:
    if window < 1 or window % 2 == 0:
        raise ValueError("window must be a positive odd integer")
    v = np.asarray(values, dtype=np.float64)
    ok = np.isfinite(v)
    k = np.ones(window)
    s = np.convolve(np.where(ok, v, 0.0), k, mode="same")
    n = np.convolve(ok.astype(np.float64), k, mode="same")
    with np.errstate(invalid="ignore", divide="ignore"):
        out = s / n
    out[n == 0] = np.nan
    return out


def binned_mean(sums: np.ndarray, counts: np.ndarray, bin_size: int) -> list[dict[str, float | int]]:
    out = []
    for a in range(0, len(sums), bin_size):
        b = min(a + bin_size, len(sums))
        n = int(counts[a:b].sum())
        out.append({"start": a, "end": b, "tokens": n, "cross_entropy": float(sums[a:b].sum() / n) if n else float("nan")})
    return out


class PerPositionLoss:
    def __init__(self, max_positions: int) -> None:
        self.sums = np.zeros(max_positions, dtype=np.float64)
        self.counts = np.zeros(max_positions, dtype=np.int64)

    def add(self, nll: Tensor | np.ndarray, start: int) -> None:
        v = nll.detach().float().cpu().numpy() if isinstance(nll, Tensor) else np.asarray(nll, dtype=np.float64)
        end = start + len(v)
        if end > len(self.sums):
            raise ValueError(f"positions up to {end} exceed max_positions {len(self.sums)}")
        self.sums[start:end] += v
        self.counts[start:end] += 1

    @property
    def tokens(self) -> int:
        return int(self.counts.sum())

    def cross_entropy(self) -> float:
        return float(self.sums.sum() / max(self.tokens, 1))

    def mean_by_position(self) -> np.ndarray:
        with np.errstate(invalid="ignore", divide="ignore"):
            m = self.sums / self.counts
        m[self.counts == 0] = np.nan
        return m

    def to_dict(self, *, ma_window: int = 101, bin_size: int = 1024) -> dict[str, Any]:
        mean = self.mean_by_position()
        clean = lambda xs: [None if not np.isfinite(x) else float(x) for x in xs]  # noqa: E731
        return {"cross_entropy": self.cross_entropy(), "tokens": self.tokens, "max_positions": len(self.sums),
                "ma_window": ma_window, "mean_by_position": clean(mean),
                "moving_average": clean(moving_average(mean, window=ma_window)),
                "bins": binned_mean(self.sums, self.counts, bin_size)}
