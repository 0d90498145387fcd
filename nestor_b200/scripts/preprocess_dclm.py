"""Tokenise a local DCLM-baseline copy (``global-shard_XX_of_10/local-shard_Y_of_10/shard_*.jsonl.zst``) into one
flat token ``.bin`` + ``.meta.json`` (the pretraining corpus; a held-out split is the same call on global shards
the training corpus never read).

``python -m nestor_b200.scripts.preprocess_dclm --dclm-root /data/dclm-baseline-1.0 --out data/dclm/dclm_train.bin
--target-tokens 11_000_000_000 --workers 48``. Shards are read in sorted order from the chosen global shards until
the token target is met; tokenisation and the output format are those of ``preprocess_text_bin``
(reference: ``scripts/preprocess_dclm.py``).
"""

from __future__ import annotations

import argparse
import multiprocessing as mp
from pathlib import Path

from nestor_b200.scripts import preprocess_text_bin


def shard_files(root: Path, global_shards: list[int] | None, file_limit: int | None) -> list[Path]:
    files: list[Path] = []
    for g in sorted(root.glob("global-shard_*_of_*")):
        index = int(g.name.split("_")[1])
        if global_shards is not None and index not in global_shards:
            continue
        files += sorted(g.glob("local-shard_*_of_*/shard_*.jsonl.zst"))
    return files[:file_limit] if file_limit else files


def main(argv: list[str] | None = None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--dclm-root", type=Path, required=True)
    ap.add_argument("--out", type=Path, required=True)
    ap.add_argument("--target-tokens", type=int, default=None)
    ap.add_argument("--global-shards", type=int, nargs="*", default=None, help="global shard numbers to read (default: all)")
    ap.add_argument("--file-limit", type=int, default=None)
    ap.add_argument("--tokenizer", default="cl100k_base")
    ap.add_argument("--workers", type=int, default=max(1, (mp.cpu_count() or 2) - 1))
    a = ap.parse_args(argv)
    files = shard_files(a.dclm_root, a.global_shards, a.file_limit)
    if not files:
        raise SystemExit(f"no shard_*.jsonl.zst files under {a.dclm_root}")
    args = [*map(str, files), "--output", str(a.out), "--tokenizer", a.tokenizer, "--workers", str(a.workers)]
    if a.target_tokens is not None:
        args += ["--max-tokens", str(a.target_tokens)]
    preprocess_text_bin.main(args)


if __name__ == "__main__":
    main()
