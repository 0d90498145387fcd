"""Held-out cross-entropy of a checkpoint over contiguous windows of a token ``.bin``.

fp32 by default (the published numbers are fp32 evaluations); the file is read as stored, without
the training loader's end-of-text remap (reference ``scripts/eval_heldout.py:29-93``).
"""

from __future__ import annotations

import argparse
import json
import math
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F

from nestor_b200.data.documents import open_token_bin
from nestor_b200.eval.loading import load_experiment_checkpoint


@torch.no_grad()
def heldout_cross_entropy(model, tokens: np.ndarray, block_size: int, device, batch: int = 1, max_windows: int | None = None) -> dict:
    n = len(tokens) // block_size
    if max_windows:
        n = min(n, max_windows)
    total, count = 0.0, 0
    model.fused_head = False
    for a in range(0, n, batch):
        rows = [np.asarray(tokens[i * block_size : (i + 1) * block_size], dtype=np.int64) for i in range(a, min(n, a + batch))]
        ids = torch.from_numpy(np.stack(rows)).to(device)
        logits = model(ids).pred[:, :-1].float()
        total += float(F.cross_entropy(logits.reshape(-1, logits.shape[-1]), ids[:, 1:].reshape(-1), reduction="sum"))
        count += ids.shape[0] * (ids.shape[1] - 1)
    ce = total / max(count, 1)
    return {"cross_entropy": ce, "perplexity": math.exp(min(ce, 50)), "tokens": count, "windows": n}


def main(argv: list[str] | None = None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--experiment", required=True); ap.add_argument("--checkpoint", type=Path, required=True)
    ap.add_argument("--data", type=Path, required=True); ap.add_argument("--block-size", type=int, default=4096)
    ap.add_argument("--batch", type=int, default=1); ap.add_argument("--max-windows", type=int, default=None)
    ap.add_argument("--bf16", action="store_true"); ap.add_argument("--ema", action="store_true")
    ap.add_argument("--output", type=Path, default=None)
    a = ap.parse_args(argv)
    device = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    model, info = load_experiment_checkpoint(a.experiment, a.checkpoint, device=device,
                                             dtype=torch.bfloat16 if a.bf16 else torch.float32, use_ema=a.ema)
    tokens, _ = open_token_bin(a.data)
    res = {**heldout_cross_entropy(model, tokens, a.block_size, device, a.batch, a.max_windows), **info,
           "experiment": a.experiment, "data": str(a.data)}
    print(json.dumps(res, indent=2))
    if a.output:
        a.output.write_text(json.dumps(res, indent=2))


if __name__ == "__main__":
    main()
