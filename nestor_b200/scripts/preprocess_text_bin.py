"""Tokenise text shards (parquet / jsonl[.gz|.zst] / txt) into a flat uint32 token ``.bin`` + ``.meta.json``.

Documents are encoded with tiktoken in a worker pool, filtered by ``--min-doc-tokens`` /
``--max-doc-tokens``, and written back to back, each followed by the end-of-text id. The same tool
serves the DCLM pretraining corpus and the domain corpora (reference: ``scripts/preprocess_dclm.py``,
``scripts/preprocess_text_bin.py``).
"""

from __future__ import annotations

import argparse
import multiprocessing as mp
from pathlib import Path

from nestor_b200.data.documents import encode_documents, init_tokenizer_worker, iter_document_texts, write_bin_meta


def batches(paths: list[Path], text_key: str, size: int):
    buf: list[str] = []
    for p in paths:
        for text in iter_document_texts(p, text_key):
            buf.append(text)
            if len(buf) >= size:
                yield buf
                buf = []
    if buf:
        yield buf


def main(argv: list[str] | None = None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("inputs", nargs="+", type=Path, help="input files or directories")
    ap.add_argument("--output", type=Path, required=True)
    ap.add_argument("--tokenizer", default="cl100k_base")
    ap.add_argument("--text-key", default="text")
    ap.add_argument("--min-doc-tokens", type=int, default=0)
    ap.add_argument("--max-doc-tokens", type=int, default=None)
    ap.add_argument("--max-tokens", type=int, default=None, help="stop after this many tokens")
    ap.add_argument("--workers", type=int, default=max(1, (mp.cpu_count() or 2) - 1))
    ap.add_argument("--batch-docs", type=int, default=256)
    a = ap.parse_args(argv)
    files: list[Path] = []
    for p in a.inputs:
        files += sorted(q for q in p.rglob("*") if q.is_file()) if p.is_dir() else [p]
    a.output.parent.mkdir(parents=True, exist_ok=True)
    tokens = docs = 0
    init = (a.tokenizer, a.min_doc_tokens, a.max_doc_tokens)
    # fresh interpreters for the workers: forking a process that already runs library threads can deadlock the child
    ctx = mp.get_context("spawn")
    with open(a.output, "wb") as out, ctx.Pool(a.workers, initializer=init_tokenizer_worker, initargs=init) as pool:
        for ids, kept in pool.imap(encode_documents, batches(files, a.text_key, a.batch_docs)):
            ids.tofile(out)
            tokens += int(ids.size)
            docs += kept
            if a.max_tokens is not None and tokens >= a.max_tokens:
                break
    write_bin_meta(a.output, num_tokens=tokens, num_docs=docs, tokenizer_name=a.tokenizer,
                   extra={"min_doc_tokens": a.min_doc_tokens, "max_doc_tokens": a.max_doc_tokens})
    print(f"wrote {a.output}: {tokens:,} tokens in {docs:,} documents")


if __name__ == "__main__":
    main()
